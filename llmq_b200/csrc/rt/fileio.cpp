// File <-> GPU transfers for checkpoints and weight import, and a memory-mapped output file shared by ranks.
//
// Reads go through two pinned staging chunks so that the pread of chunk i+1 overlaps the H2D copy of chunk i
// (the reference's fallback path uses one 1 MiB pinned chunk and synchronous copies,
// src/utilities/cu_file_fallback.cpp:33-73; its GDS path needs cuFile, which is optional there and absent here).
// Writes copy device memory into a caller-visible mapping of the output file (D2H straight into the page
// cache), the same idea as the reference's safetensors writer (src/utilities/safetensors.cpp:197-339).
#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {
constexpr size_t kChunk = 8u << 20;

struct Staging {
    void* buf[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool ok = false;
    Staging() {
        ok = cudaMallocHost(&buf[0], kChunk) == cudaSuccess && cudaMallocHost(&buf[1], kChunk) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming) == cudaSuccess;
    }
    ~Staging() {
        for (int i = 0; i < 2; ++i) {
            if (buf[i]) cudaFreeHost(buf[i]);
            if (done[i]) cudaEventDestroy(done[i]);
        }
    }
};
}  // namespace

extern "C" {

// Reads nbytes at `offset` of the file into `dst`.  dst_is_device != 0: device memory (pinned double-buffered
// staging, asynchronous copies on `stream`, synchronised before returning); otherwise plain host memory.
// Returns 0, -errno for I/O errors, or a positive CUDA error code.
int llmq_rt_read_file(const char* path, long long offset, long long nbytes, void* dst, int dst_is_device, cudaStream_t stream) {
    int fd = ::open(path, O_RDONLY);
    if (fd < 0) return -errno;
    int rc = 0;
    if (!dst_is_device) {
        long long done = 0;
        while (done < nbytes) {
            ssize_t r = pread(fd, static_cast<char*>(dst) + done, static_cast<size_t>(nbytes - done), offset + done);
            if (r <= 0) { rc = r < 0 ? -errno : -EIO; break; }
            done += r;
        }
        ::close(fd);
        return rc;
    }
    Staging st;
    if (!st.ok) { ::close(fd); return static_cast<int>(cudaErrorMemoryAllocation); }
    long long done = 0;
    int slot = 0;
    bool used[2] = {false, false};
    while (done < nbytes && rc == 0) {
        size_t n = static_cast<size_t>(std::min<long long>(kChunk, nbytes - done));
        if (used[slot]) {
            cudaError_t e = cudaEventSynchronize(st.done[slot]);
            if (e != cudaSuccess) { rc = static_cast<int>(e); break; }
        }
        size_t got = 0;
        while (got < n) {
            ssize_t r = pread(fd, static_cast<char*>(st.buf[slot]) + got, n - got, offset + done + static_cast<long long>(got));
            if (r <= 0) { rc = r < 0 ? -errno : -EIO; break; }
            got += static_cast<size_t>(r);
        }
        if (rc) break;
        cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dst) + done, st.buf[slot], n, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaEventRecord(st.done[slot], stream);
        if (e != cudaSuccess) { rc = static_cast<int>(e); break; }
        used[slot] = true;
        done += static_cast<long long>(n);
        slot ^= 1;
    }
    cudaError_t e = cudaStreamSynchronize(stream);
    if (rc == 0 && e != cudaSuccess) rc = static_cast<int>(e);
    ::close(fd);
    return rc;
}

// Creates (create != 0: truncates to `size`) or opens a file and maps it read-write.  Returns the mapping or null.
void* llmq_rt_map_file(const char* path, long long size, int create) {
    int fd = ::open(path, create ? (O_RDWR | O_CREAT | O_TRUNC) : O_RDWR, 0644);
    if (fd < 0) return nullptr;
    if (create && ftruncate(fd, size) != 0) { ::close(fd); return nullptr; }
    void* m = mmap(nullptr, static_cast<size_t>(size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    return m == MAP_FAILED ? nullptr : m;
}
int llmq_rt_unmap_file(void* map, long long size, int sync) {
    if (sync && msync(map, static_cast<size_t>(size), MS_SYNC) != 0) return -errno;
    return munmap(map, static_cast<size_t>(size)) == 0 ? 0 : -errno;
}
// Copies nbytes from `src` (device or host) to map + offset.
int llmq_rt_write_to_map(void* map, long long offset, const void* src, long long nbytes, int src_is_device, cudaStream_t stream) {
    char* dst = static_cast<char*>(map) + offset;
    if (!src_is_device) { std::memcpy(dst, src, static_cast<size_t>(nbytes)); return 0; }
    cudaError_t e = cudaMemcpyAsync(dst, src, static_cast<size_t>(nbytes), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return static_cast<int>(e);
}

}  // extern "C"
