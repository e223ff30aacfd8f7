// LIFO bump allocator over one backing buffer, for step-scoped temporaries.
//
// Counterpart of DeviceMemoryStack (src/utilities/stack.cpp:13-56 of the reference): allocations are 4 KiB
// aligned offsets into a buffer owned by the caller, frees must come in reverse order, the high-water mark is
// tracked, and a dry-run instance (no backing memory, 1 TiB capacity) is used to size the real buffer by
// replaying the allocation pattern of one step.  The library only does the bookkeeping; the Python side turns
// offsets into tensor views of its backing tensor.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace {
constexpr long long kAlign = 4096;

struct Entry {
    long long offset, bytes;
    std::string name;
};
struct Stack {
    long long capacity = 0, top = 0, high_water = 0;
    bool dry_run = false;
    std::vector<Entry> live;
    std::vector<Entry> high_water_set;     // what was live when the high-water mark was reached
    std::string error;
};
}  // namespace

extern "C" {

void* llmq_stack_create(long long capacity_bytes, int dry_run) {
    auto* s = new Stack();
    s->dry_run = dry_run != 0;
    s->capacity = s->dry_run ? (1LL << 40) : capacity_bytes;
    return s;
}
void llmq_stack_destroy(void* h) { delete static_cast<Stack*>(h); }

// Returns the byte offset of the new block, or -1 (see llmq_stack_error).
long long llmq_stack_alloc(void* h, long long bytes, const char* name) {
    auto* s = static_cast<Stack*>(h);
    long long rounded = (bytes + kAlign - 1) / kAlign * kAlign;
    if (s->top + rounded > s->capacity) {
        s->error = "stack overflow allocating '" + std::string(name ? name : "?") + "': need " + std::to_string(rounded) +
                   " bytes, " + std::to_string(s->capacity - s->top) + " free of " + std::to_string(s->capacity);
        return -1;
    }
    long long off = s->top;
    s->live.push_back({off, rounded, name ? name : ""});
    s->top += rounded;
    if (s->top > s->high_water) {
        s->high_water = s->top;
        s->high_water_set = s->live;
    }
    return off;
}
// Frees the most recent allocation; `offset` must be its offset (LIFO order is enforced).
int llmq_stack_free(void* h, long long offset) {
    auto* s = static_cast<Stack*>(h);
    if (s->live.empty()) { s->error = "free on an empty stack"; return -1; }
    if (s->live.back().offset != offset) {
        s->error = "out-of-order free: top of stack is '" + s->live.back().name + "'";
        return -1;
    }
    s->top = s->live.back().offset;
    s->live.pop_back();
    return 0;
}
long long llmq_stack_used(void* h) { return static_cast<Stack*>(h)->top; }
long long llmq_stack_high_water(void* h) { return static_cast<Stack*>(h)->high_water; }
long long llmq_stack_capacity(void* h) { return static_cast<Stack*>(h)->capacity; }
int llmq_stack_live_count(void* h) { return static_cast<int>(static_cast<Stack*>(h)->live.size()); }
const char* llmq_stack_error(void* h) { return static_cast<Stack*>(h)->error.c_str(); }
// Writes "name:bytes;name:bytes;..." of the allocations that were live at the high-water mark.
int llmq_stack_high_water_report(void* h, char* out, int out_bytes) {
    auto* s = static_cast<Stack*>(h);
    std::string r;
    for (auto& e : s->high_water_set) r += e.name + ":" + std::to_string(e.bytes) + ";";
    if (static_cast<int>(r.size()) + 1 > out_bytes) return -1;
    std::memcpy(out, r.c_str(), r.size() + 1);
    return static_cast<int>(r.size());
}

}  // extern "C"
