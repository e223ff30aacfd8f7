// Page-locked host memory with explicit flags, for offloaded tensors.
//
// The reference allocates offloaded state with cudaHostAlloc and, on request, as write-combined memory
// (`--write-combined`, src/utilities/allocator.cpp:57-70): the CPU never reads those tensors during training, and
// write-combined pages skip the CPU caches, which can speed up PCIe transfers.  Every allocation is also mapped into
// the device address space (the default under unified addressing), so kernels can use the same pointer directly
// (`--use-zero-copy`).
#include <cuda_runtime.h>

extern "C" {

// Returns the host pointer (also valid on the device), or null when the allocation failed or no CUDA device exists.
void* llmq_host_alloc(long long bytes, int write_combined) {
    if (bytes <= 0) return nullptr;
    void* p = nullptr;
    unsigned int flags = cudaHostAllocMapped | cudaHostAllocPortable;
    if (write_combined) flags |= cudaHostAllocWriteCombined;
    if (cudaHostAlloc(&p, static_cast<size_t>(bytes), flags) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

int llmq_host_free(void* p) {
    if (!p) return 0;
    return static_cast<int>(cudaFreeHost(p));
}

}  // extern "C"
