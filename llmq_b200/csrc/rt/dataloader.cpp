// Native streaming loader for pre-tokenised BIN.TOK files.
//
// File format (same as the reference, scripts/tokenize_data.py:60-128 and src/training/dataloader.cpp:84-118):
// a 1024-byte header "BIN.TOK\n" + int32 {version, bytes_per_token (4), n_tokens, vocab_size, has_masks},
// then int32 tokens, then an optional little-endian packed bit mask (1 = train on this target).
//
// Behaviour kept: sequences are non-overlapping chunks of seq_len tokens, targets are the inputs shifted
// by one token, masked targets become -100, files and chunks are visited in a deterministic pseudo-random
// order that depends only on (seed, epoch, file), rank r takes chunks r, r + world, r + 2*world, ...; the
// position is (seed, epoch, file_index, chunk_index) and can be saved / restored.
//
// Design: every file is mmap'ed read-only, so a batch is a handful of memcpy calls out of the page cache
// straight into the caller's (pinned) buffers; there is no stream state to seek around.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

struct TokenFile {
    std::string name;
    int version = 0;
    long long n_tokens = 0;
    int vocab = 0;
    bool has_masks = false;
    const uint8_t* map = nullptr;
    size_t map_bytes = 0;
};

uint64_t splitmix64(uint64_t& x) {
    uint64_t z = (x += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

template <typename T>
void shuffle(std::vector<T>& v, uint64_t seed, uint64_t a, uint64_t b) {
    uint64_t s = seed * 0x2545F4914F6CDD1Dull + a * 0x9E3779B97F4A7C15ull + b * 0xD6E8FEB86659FD93ull + 1;
    for (size_t i = v.size(); i > 1; --i) {
        size_t j = static_cast<size_t>(splitmix64(s) % i);
        std::swap(v[i - 1], v[j]);
    }
}

struct Loader {
    std::vector<TokenFile> files;
    std::vector<int> file_order;
    std::vector<int> chunk_order;
    int seq_len = 0, rank = 0, world = 1;
    uint64_t seed = 0;
    int epoch = -1, file_index = -1;
    long long chunk_index = 0;          // includes the rank offset
    long long total_tokens = 0, total_chunks = 0;
    std::string error;

    const TokenFile& cur() const { return files[file_order[file_index]]; }

    void shuffle_files() {
        file_order.resize(files.size());
        for (size_t i = 0; i < files.size(); ++i) file_order[i] = static_cast<int>(i);
        shuffle(file_order, seed, static_cast<uint64_t>(epoch), 0x73653753ull);
    }
    void shuffle_chunks() {
        long long n = (cur().n_tokens - 1) / seq_len;
        chunk_order.resize(static_cast<size_t>(n));
        for (long long i = 0; i < n; ++i) chunk_order[static_cast<size_t>(i)] = static_cast<int>(i);
        shuffle(chunk_order, seed, static_cast<uint64_t>(epoch), static_cast<uint64_t>(file_order[file_index]) + 1);
    }
    bool advance_file() {
        ++file_index;
        if (file_index >= static_cast<int>(files.size())) return false;
        shuffle_chunks();
        chunk_index = rank;
        return true;
    }
    void advance_epoch() {
        ++epoch;
        shuffle_files();
        file_index = -1;
        advance_file();
    }
    bool has_next(int n) const {
        if (file_index != static_cast<int>(files.size()) - 1) return true;
        return chunk_index - rank + static_cast<long long>(n) * world <= static_cast<long long>(chunk_order.size());
    }
    bool load_seq(int32_t* inputs, int32_t* targets) {
        // a round needs one chunk for every rank; a file's ragged tail is skipped by all ranks together
        while (chunk_index - rank + world > static_cast<long long>(chunk_order.size())) {
            if (!advance_file()) { error = "No more files to load"; return false; }
        }
        const TokenFile& f = cur();
        const long long pos = static_cast<long long>(seq_len) * chunk_order[static_cast<size_t>(chunk_index)];
        const int32_t* tok = reinterpret_cast<const int32_t*>(f.map + 1024);
        std::memcpy(inputs, tok + pos, sizeof(int32_t) * seq_len);
        std::memcpy(targets, tok + pos + 1, sizeof(int32_t) * seq_len);
        if (f.has_masks) {
            const uint8_t* masks = f.map + 1024 + 4 * f.n_tokens;
            for (int i = 0; i < seq_len; ++i) {
                long long bit = pos + i;
                if (!((masks[bit >> 3] >> (bit & 7)) & 1)) targets[i] = -100;
            }
        }
        chunk_index += world;
        return true;
    }
};

bool open_file(const char* path, TokenFile& f, std::string& err) {
    int fd = ::open(path, O_RDONLY);
    if (fd < 0) { err = std::string("Could not open token file: ") + path; return false; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 1024) { ::close(fd); err = std::string("Token file too small: ") + path; return false; }
    void* m = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) { err = std::string("mmap failed for ") + path; return false; }
    const int32_t* h = static_cast<const int32_t*>(m);
    if (std::memcmp(m, "BIN.TOK\n", 8) != 0) { munmap(m, st.st_size); err = std::string("Invalid token file: ") + path; return false; }
    f.name = path;
    f.version = h[2];
    if (f.version != 1 && f.version != 2) { munmap(m, st.st_size); err = "Unsupported token file version"; return false; }
    if (h[3] != 4) { munmap(m, st.st_size); err = "Unsupported bytes per token"; return false; }
    f.n_tokens = h[4];
    f.vocab = f.version == 2 ? h[5] : 0;
    f.has_masks = h[6] == 1;
    f.map = static_cast<const uint8_t*>(m);
    f.map_bytes = static_cast<size_t>(st.st_size);
    size_t need = 1024 + 4 * static_cast<size_t>(f.n_tokens) + (f.has_masks ? (static_cast<size_t>(f.n_tokens) + 7) / 8 : 0);
    if (f.map_bytes < need) { munmap(m, st.st_size); err = std::string("Truncated token file: ") + path; return false; }
    return true;
}

}  // namespace

extern "C" {

// paths: n_files null-terminated strings.  Returns an opaque handle or null (then *err_out, if given, holds a
// message valid until the next call on this thread).
void* llmq_dl_create(const char** paths, int n_files, int seq_len, int rank, int world, unsigned long long seed, const char** err_out) {
    static thread_local std::string last_error;
    auto* L = new Loader();
    L->seq_len = seq_len; L->rank = rank; L->world = world; L->seed = seed;
    if (n_files <= 0) { last_error = "Empty list of token files provided"; if (err_out) *err_out = last_error.c_str(); delete L; return nullptr; }
    for (int i = 0; i < n_files; ++i) {
        TokenFile f;
        if (!open_file(paths[i], f, last_error)) { if (err_out) *err_out = last_error.c_str(); delete L; return nullptr; }
        L->files.push_back(f);
    }
    for (auto& f : L->files) {
        if (f.vocab != L->files[0].vocab) { last_error = "Inconsistent vocabulary sizes in " + f.name; if (err_out) *err_out = last_error.c_str(); delete L; return nullptr; }
        L->total_tokens += f.n_tokens;
        L->total_chunks += (f.n_tokens - 1) / seq_len;
    }
    L->advance_epoch();
    return L;
}

void llmq_dl_destroy(void* h) {
    auto* L = static_cast<Loader*>(h);
    if (!L) return;
    for (auto& f : L->files) if (f.map) munmap(const_cast<uint8_t*>(f.map), f.map_bytes);
    delete L;
}

// inputs / targets: batch * seq_len int32 each.  Returns 0, or -1 when the data ran out (see llmq_dl_error).
int llmq_dl_load_batch(void* h, int32_t* inputs, int32_t* targets, int batch) {
    auto* L = static_cast<Loader*>(h);
    for (int b = 0; b < batch; ++b)
        if (!L->load_seq(inputs + static_cast<long long>(b) * L->seq_len, targets + static_cast<long long>(b) * L->seq_len)) return -1;
    return 0;
}
const char* llmq_dl_error(void* h) { return static_cast<Loader*>(h)->error.c_str(); }
int llmq_dl_has_next(void* h, int n) { return static_cast<Loader*>(h)->has_next(n) ? 1 : 0; }
void llmq_dl_advance_epoch(void* h) { static_cast<Loader*>(h)->advance_epoch(); }

void llmq_dl_set_state(void* h, unsigned long long seed, int epoch, int file_index, long long chunk_index) {
    auto* L = static_cast<Loader*>(h);
    L->seed = seed;
    L->epoch = epoch;
    L->shuffle_files();
    L->file_index = file_index;
    if (file_index >= 0 && file_index < static_cast<int>(L->files.size())) L->shuffle_chunks();
    L->chunk_index = chunk_index + L->rank;
}
// out: {seed, epoch, file_index, chunk_index (without rank offset), total_tokens, total_chunks, vocab, n_files}
void llmq_dl_get_state(void* h, long long* out) {
    auto* L = static_cast<Loader*>(h);
    out[0] = static_cast<long long>(L->seed); out[1] = L->epoch; out[2] = L->file_index; out[3] = L->chunk_index - L->rank;
    out[4] = L->total_tokens; out[5] = L->total_chunks; out[6] = L->files[0].vocab; out[7] = static_cast<long long>(L->files.size());
}
const char* llmq_dl_current_file(void* h) {
    auto* L = static_cast<Loader*>(h);
    if (L->file_index < 0 || L->file_index >= static_cast<int>(L->files.size())) return "";
    return L->cur().name.c_str();
}
double llmq_dl_progress(void* h) {
    auto* L = static_cast<Loader*>(h);
    long long t = 0;
    for (int i = 0; i < L->file_index && i < static_cast<int>(L->files.size()); ++i) t += L->files[L->file_order[i]].n_tokens;
    t += (L->chunk_index - L->rank) * L->seq_len;
    return 100.0 * static_cast<double>(t) / static_cast<double>(L->total_tokens > 0 ? L->total_tokens : 1);
}

}  // extern "C"
