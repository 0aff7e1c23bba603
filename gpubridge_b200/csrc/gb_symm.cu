// Symmetric memory: one workspace per rank, mapped into every peer of the team.
//
// The default mapping uses CUDA IPC: the owner allocates with cudaMalloc and exports a
// 64-byte handle, which the ranks exchange through the job's store; every peer opens it
// and gets a pointer it can use in kernels (loads and stores travel over NVLink).  The
// control block (grid barrier, sequence numbers, abort word) is ordinary device memory and
// the status block is mapped host memory, so the host can read a failure without
// synchronising the device.
//
// Nothing here is called on a hot path: a team maps its workspaces once.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" {

const char* gb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

int gb_device_count(int* count) { return (int)cudaGetDeviceCount(count); }

// A zeroed device allocation of `bytes` on the current device.
int gb_symm_alloc(size_t bytes, void** ptr) {
    cudaError_t err = cudaMalloc(ptr, bytes);
    if (err != cudaSuccess) return (int)err;
    err = cudaMemset(*ptr, 0, bytes);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaDeviceSynchronize();
}

int gb_device_synchronize() { return (int)cudaDeviceSynchronize(); }

int gb_symm_free(void* ptr) { return (int)cudaFree(ptr); }

int gb_symm_export(void* ptr, unsigned char* handle64) {
    cudaIpcMemHandle_t h;
    cudaError_t err = cudaIpcGetMemHandle(&h, ptr);
    if (err != cudaSuccess) return (int)err;
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    memcpy(handle64, &h, sizeof(h));
    return 0;
}

int gb_symm_import(const unsigned char* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int gb_symm_unmap(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

// Whether `device` can address `peer`'s memory directly.
int gb_can_access_peer(int device, int peer, int* yes) {
    return (int)cudaDeviceCanAccessPeer(yes, device, peer);
}

// Mapped, zeroed host memory for the status words; the device uses the same address.
int gb_status_alloc(size_t bytes, void** host) {
    cudaError_t err = cudaHostAlloc(host, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    if (err != cudaSuccess) return (int)err;
    memset(*host, 0, bytes);
    return 0;
}

int gb_status_free(void* host) { return (int)cudaFreeHost(host); }

int gb_memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) {
    return (int)cudaMemsetAsync(ptr, value, bytes, stream);
}

// Copy `bytes` of device memory into pinned host memory on `stream` (the barrier timestamps of
// the last collective, for observers).
int gb_copy_to_host(void* host, const void* device, size_t bytes, cudaStream_t stream) {
    return (int)cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, stream);
}

}  // extern "C"
