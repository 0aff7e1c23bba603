// NVLink multicast objects and the memory bound to them, created by the fabric itself.
//
// A multicast object joins one physical allocation per GPU of a group.  Mapped into a
// process it gives a "multicast address": a multimem.ld_reduce on it returns the sum of that
// address over every GPU of the group, computed inside the NVSwitch, and a multimem.st writes
// every GPU's copy at once.  The in-switch all-reduce (gb_switch.cu) stages through such
// memory.  One group is the team, and - for a team of several islands - one more per island,
// so that the island step of the hierarchical all-reduce runs through the switch too.
//
// Everything here goes through the CUDA driver API (virtual memory management), looked up
// at run time with cudaGetDriverEntryPoint: the library links against the runtime only.
// Handles cross process boundaries as POSIX file descriptors; passing the descriptor to the
// other ranks (a Unix socket) is the caller's business.  Nothing here is on a hot path.
//
// Call order for a group (every step by every member unless stated):
//   gb_mc_create (one member) -> gb_vmm_export -> [descriptor to the others] -> gb_vmm_import
//   gb_mc_add_device              ... all members, and all of them before anybody binds
//   gb_vmm_create + gb_mc_bind    ... the member's own memory at offset 0 of the object
//   gb_vmm_map (the memory)  -> the local address;  gb_vmm_map (the object) -> the multicast address
// and the reverse to tear down: gb_vmm_unmap both, gb_mc_unbind, gb_vmm_release both.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace {

template <typename F> F driver(const char* name) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
        return nullptr;
    return reinterpret_cast<F>(ptr);
}

// Error codes of this file: a CUresult (> 0), or -1 when the driver lacks the entry point.
#define GB_DRIVER(var, type, name)                  \
    static type var = driver<type>(name);           \
    if (var == nullptr) return -1

typedef CUresult (*FnDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
typedef CUresult (*FnMcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
typedef CUresult (*FnMcAddDevice)(CUmemGenericAllocationHandle, CUdevice);
typedef CUresult (*FnMcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                                size_t, size_t, unsigned long long);
typedef CUresult (*FnMcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
typedef CUresult (*FnMcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
typedef CUresult (*FnMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                                unsigned long long);
typedef CUresult (*FnMemRelease)(CUmemGenericAllocationHandle);
typedef CUresult (*FnMemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                unsigned long long);
typedef CUresult (*FnMemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
typedef CUresult (*FnMemReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*FnMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                             unsigned long long);
typedef CUresult (*FnMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
typedef CUresult (*FnMemUnmap)(CUdeviceptr, size_t);
typedef CUresult (*FnMemAddressFree)(CUdeviceptr, size_t);
typedef CUresult (*FnMemGranularity)(size_t*, const CUmemAllocationProp*,
                                     CUmemAllocationGranularity_flags);
typedef CUresult (*FnGetErrorString)(CUresult, const char**);

CUmulticastObjectProp object_prop(int devices, size_t bytes) {
    CUmulticastObjectProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.numDevices = (unsigned)devices;
    prop.size = bytes;
    prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

CUmemAllocationProp memory_prop(int device) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

}  // namespace

extern "C" {

// Text of a code returned by the functions of this file.
const char* gb_mc_error_string(int code) {
    if (code == -1) return "the CUDA driver lacks a virtual-memory or multicast entry point";
    static FnGetErrorString text = driver<FnGetErrorString>("cuGetErrorString");
    const char* out = nullptr;
    if (text != nullptr && text((CUresult)code, &out) == CUDA_SUCCESS && out != nullptr) return out;
    return "unknown CUDA driver error";
}

// Whether `device` can join a multicast object (NVSwitch fabric with multicast enabled).
int gb_mc_supported(int device, int* yes) {
    *yes = 0;
    GB_DRIVER(attribute, FnDeviceGetAttribute, "cuDeviceGetAttribute");
    int vmm = 0, mc = 0;
    CUresult err = attribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device);
    if (err != CUDA_SUCCESS) return (int)err;
    err = attribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device);
    if (err != CUDA_SUCCESS) return (int)err;
    *yes = vmm && mc;
    return 0;
}

// The size granularity of an object of `devices` GPUs: sizes, and the memory bound to it, are
// multiples of it (it is at least the allocation granularity of the memory).
int gb_mc_granularity(int device, int devices, size_t bytes, size_t* granularity) {
    GB_DRIVER(mc_gran, FnMcGranularity, "cuMulticastGetGranularity");
    GB_DRIVER(mem_gran, FnMemGranularity, "cuMemGetAllocationGranularity");
    const CUmulticastObjectProp prop = object_prop(devices, bytes);
    size_t a = 0, b = 0;
    CUresult err = mc_gran(&a, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (err != CUDA_SUCCESS) return (int)err;
    const CUmemAllocationProp mem = memory_prop(device);
    err = mem_gran(&b, &mem, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (err != CUDA_SUCCESS) return (int)err;
    *granularity = a > b ? a : b;
    return 0;
}

int gb_mc_create(int devices, size_t bytes, unsigned long long* object) {
    GB_DRIVER(create, FnMcCreate, "cuMulticastCreate");
    const CUmulticastObjectProp prop = object_prop(devices, bytes);
    CUmemGenericAllocationHandle handle = 0;
    const CUresult err = create(&handle, &prop);
    *object = (unsigned long long)handle;
    return (int)err;
}

int gb_mc_add_device(unsigned long long object, int device) {
    GB_DRIVER(add, FnMcAddDevice, "cuMulticastAddDevice");
    return (int)add((CUmemGenericAllocationHandle)object, (CUdevice)device);
}

// Bind `bytes` of `memory` (from its start) at the start of the object.
int gb_mc_bind(unsigned long long object, unsigned long long memory, size_t bytes) {
    GB_DRIVER(bind, FnMcBindMem, "cuMulticastBindMem");
    return (int)bind((CUmemGenericAllocationHandle)object, 0,
                     (CUmemGenericAllocationHandle)memory, 0, bytes, 0);
}

int gb_mc_unbind(unsigned long long object, int device, size_t bytes) {
    GB_DRIVER(unbind, FnMcUnbind, "cuMulticastUnbind");
    return (int)unbind((CUmemGenericAllocationHandle)object, (CUdevice)device, 0, bytes);
}

// `bytes` of physical memory on `device` (a multiple of the granularity).
int gb_vmm_create(int device, size_t bytes, unsigned long long* memory) {
    GB_DRIVER(create, FnMemCreate, "cuMemCreate");
    const CUmemAllocationProp prop = memory_prop(device);
    CUmemGenericAllocationHandle handle = 0;
    const CUresult err = create(&handle, bytes, &prop, 0);
    *memory = (unsigned long long)handle;
    return (int)err;
}

int gb_vmm_release(unsigned long long handle) {
    GB_DRIVER(release, FnMemRelease, "cuMemRelease");
    return (int)release((CUmemGenericAllocationHandle)handle);
}

// A file descriptor for a memory or multicast handle; the caller closes it after sending it.
int gb_vmm_export(unsigned long long handle, int* fd) {
    GB_DRIVER(to_fd, FnMemExport, "cuMemExportToShareableHandle");
    return (int)to_fd(fd, (CUmemGenericAllocationHandle)handle,
                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
}

int gb_vmm_import(int fd, unsigned long long* handle) {
    GB_DRIVER(from_fd, FnMemImport, "cuMemImportFromShareableHandle");
    CUmemGenericAllocationHandle out = 0;
    const CUresult err = from_fd(&out, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    *handle = (unsigned long long)out;
    return (int)err;
}

// Map a memory or multicast handle for reading and writing by `device`; `alignment`: the
// granularity.  The mapping is new address space: the same handle may be mapped twice.
int gb_vmm_map(unsigned long long handle, size_t bytes, size_t alignment, int device, void** ptr) {
    GB_DRIVER(reserve, FnMemReserve, "cuMemAddressReserve");
    GB_DRIVER(map, FnMemMap, "cuMemMap");
    GB_DRIVER(access, FnMemSetAccess, "cuMemSetAccess");
    GB_DRIVER(unmap, FnMemUnmap, "cuMemUnmap");
    GB_DRIVER(release, FnMemAddressFree, "cuMemAddressFree");
    CUdeviceptr va = 0;
    CUresult err = reserve(&va, bytes, alignment, 0, 0);
    if (err != CUDA_SUCCESS) return (int)err;
    err = map(va, bytes, 0, (CUmemGenericAllocationHandle)handle, 0);
    if (err != CUDA_SUCCESS) { release(va, bytes); return (int)err; }
    CUmemAccessDesc desc;
    memset(&desc, 0, sizeof(desc));
    desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    desc.location.id = device;
    desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    err = access(va, bytes, &desc, 1);
    if (err != CUDA_SUCCESS) { unmap(va, bytes); release(va, bytes); return (int)err; }
    *ptr = reinterpret_cast<void*>(va);
    return 0;
}

int gb_vmm_unmap(void* ptr, size_t bytes) {
    GB_DRIVER(unmap, FnMemUnmap, "cuMemUnmap");
    GB_DRIVER(release, FnMemAddressFree, "cuMemAddressFree");
    const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
    const CUresult err = unmap(va, bytes);
    if (err != CUDA_SUCCESS) return (int)err;
    return (int)release(va, bytes);
}

}  // extern "C"
