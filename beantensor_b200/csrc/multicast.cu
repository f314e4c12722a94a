// NVSwitch multicast memory for the N-sharded product: one full-size C per rank, all of them bound to one
// multicast object, so that a single multimem.st from a rank's epilogue lands in every rank's copy (the switch
// replicates it) instead of the rank sending the same bytes to each peer in turn.
//
// Host side only (CUDA virtual-memory-management and multicast driver calls). One process per GPU: the rank that
// creates the multicast object exports it as a POSIX file descriptor, the caller carries that descriptor to the other
// processes (a Unix-domain socket with SCM_RIGHTS; beantensor_b200/multicast.py does it), they import it. Every rank
// then adds its device, creates its own physical memory, binds it at offset 0 and maps two ranges: its own memory
// (ordinary loads and stores) and the multicast object (multimem stores only; nothing here ever loads through it).
// Release order matters on NVSwitch systems: every rank unmaps and unbinds while all ranks are still alive, so callers
// release behind a barrier and never leave a bound rank behind.
#include <unistd.h>

#include <cstring>
#include <mutex>

#include "btm_internal.h"

namespace btm {

namespace {

struct DriverApi {
    bool ready = false;
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
};
DriverApi g_drv;
std::mutex g_drv_mu;

template <typename F>
bool lookup(const char *name, F *fn)
{
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
        (void)cudaGetLastError();
        return false;
    }
    *fn = reinterpret_cast<F>(p);
    return true;
}

int driver()
{
    std::lock_guard<std::mutex> lock(g_drv_mu);
    if (g_drv.ready) return BTM_OK;
    bool ok = lookup("cuDeviceGet", &g_drv.DeviceGet) && lookup("cuDeviceGetAttribute", &g_drv.DeviceGetAttribute) &&
              lookup("cuMulticastCreate", &g_drv.MulticastCreate) && lookup("cuMulticastAddDevice", &g_drv.MulticastAddDevice) &&
              lookup("cuMulticastBindMem", &g_drv.MulticastBindMem) && lookup("cuMulticastUnbind", &g_drv.MulticastUnbind) &&
              lookup("cuMulticastGetGranularity", &g_drv.MulticastGetGranularity) && lookup("cuMemCreate", &g_drv.MemCreate) &&
              lookup("cuMemRelease", &g_drv.MemRelease) && lookup("cuMemExportToShareableHandle", &g_drv.MemExportToShareableHandle) &&
              lookup("cuMemImportFromShareableHandle", &g_drv.MemImportFromShareableHandle) &&
              lookup("cuMemAddressReserve", &g_drv.MemAddressReserve) && lookup("cuMemAddressFree", &g_drv.MemAddressFree) &&
              lookup("cuMemMap", &g_drv.MemMap) && lookup("cuMemUnmap", &g_drv.MemUnmap) && lookup("cuMemSetAccess", &g_drv.MemSetAccess) &&
              lookup("cuMemGetAllocationGranularity", &g_drv.MemGetAllocationGranularity);
    if (!ok) return set_error(BTM_ERR_UNSUPPORTED, "multicast memory: the driver does not export the virtual-memory / multicast entry points");
    g_drv.ready = true;
    return BTM_OK;
}

int check_cu(CUresult r, const char *what)
{
    if (r == CUDA_SUCCESS) return BTM_OK;
    if (r == CUDA_ERROR_OUT_OF_MEMORY) return set_error(BTM_ERR_OOM, "CUDA Error: out of memory (%s)", what);
    if (r == CUDA_ERROR_NOT_SUPPORTED || r == CUDA_ERROR_NOT_PERMITTED)
        return set_error(BTM_ERR_UNSUPPORTED, "multicast memory: %s is not supported or not permitted here (driver code %d)", what, (int)r);
    return set_error(BTM_ERR_CUDA, "CUDA Error: %s failed with driver code %d", what, (int)r);
}

} // namespace

} // namespace btm

using namespace btm;

struct btm_mc {
    int device;
    int nranks;
    CUdevice cu_dev;
    size_t bytes;   // rounded to the multicast granularity
    CUmemGenericAllocationHandle mc;
    CUmemGenericAllocationHandle mem;
    CUdeviceptr va_local, va_mc;
    bool have_mc, added, have_mem, bound, mapped_local, mapped_mc;
};

static CUmulticastObjectProp mc_prop(int nranks, size_t bytes)
{
    CUmulticastObjectProp p;
    memset(&p, 0, sizeof(p));
    p.numDevices = (unsigned)nranks;
    p.size = bytes;
    p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return p;
}

static int mc_begin(int device, int nranks, size_t bytes, btm_mc **out)
{
    if (!out) return set_error(BTM_ERR_INVALID, "multicast memory: null handle pointer");
    *out = nullptr;
    if (nranks < 2 || nranks > kMaxDst) return set_error(BTM_ERR_INVALID, "multicast memory: %d ranks (2 to %d are supported)", nranks, kMaxDst);
    if (bytes == 0) return set_error(BTM_ERR_INVALID, "multicast memory: zero size");
    if (!device_state(device)) return BTM_ERR_CUDA;
    int rc = driver();
    if (rc) return rc;
    CUdevice dev;
    rc = check_cu(g_drv.DeviceGet(&dev, device), "cuDeviceGet");
    if (rc) return rc;
    int supported = 0;
    rc = check_cu(g_drv.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev), "cuDeviceGetAttribute");
    if (rc) return rc;
    if (!supported) return set_error(BTM_ERR_UNSUPPORTED, "multicast memory: device %d does not support multicast objects", device);
    CUmulticastObjectProp p = mc_prop(nranks, bytes);
    size_t gran = 0;
    rc = check_cu(g_drv.MulticastGetGranularity(&gran, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (rc) return rc;
    if (gran == 0) gran = 2u << 20;
    btm_mc *h = new btm_mc();
    memset(h, 0, sizeof(*h));
    h->device = device;
    h->nranks = nranks;
    h->cu_dev = dev;
    h->bytes = (bytes + gran - 1) / gran * gran;
    *out = h;
    return BTM_OK;
}

extern "C" {

int btm_mc_supported(int device)
{
    if (!device_state(device)) return 0;
    if (driver()) return 0;
    CUdevice dev;
    int supported = 0;
    if (g_drv.DeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
    if (g_drv.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
    return supported ? 1 : 0;
}

int btm_mc_create(int device, int nranks, size_t bytes, btm_mc **out, int *export_fd)
{
    if (!export_fd) return set_error(BTM_ERR_INVALID, "multicast memory: null descriptor pointer");
    int rc = mc_begin(device, nranks, bytes, out);
    if (rc) return rc;
    btm_mc *h = *out;
    CUmulticastObjectProp p = mc_prop(nranks, h->bytes);
    rc = check_cu(g_drv.MulticastCreate(&h->mc, &p), "cuMulticastCreate");
    if (!rc) {
        h->have_mc = true;
        int fd = -1;
        rc = check_cu(g_drv.MemExportToShareableHandle(&fd, h->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
        if (!rc) *export_fd = fd;
    }
    if (rc) {
        btm_mc_release(h);
        *out = nullptr;
    }
    return rc;
}

int btm_mc_import(int device, int nranks, size_t bytes, int fd, btm_mc **out)
{
    int rc = mc_begin(device, nranks, bytes, out);
    if (rc) return rc;
    btm_mc *h = *out;
    rc = check_cu(g_drv.MemImportFromShareableHandle(&h->mc, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle");
    if (rc) {
        btm_mc_release(h);
        *out = nullptr;
        return rc;
    }
    h->have_mc = true;
    return BTM_OK;
}

int btm_mc_add_device(btm_mc *h)
{
    if (!h) return set_error(BTM_ERR_INVALID, "multicast memory: null argument");
    if (!h->have_mc || h->added) return set_error(BTM_ERR_INVALID, "multicast memory: handle is not in a state to add its device");
    if (!device_state(h->device)) return BTM_ERR_CUDA;
    int rc = check_cu(g_drv.MulticastAddDevice(h->mc, h->cu_dev), "cuMulticastAddDevice");
    if (rc) return rc;
    h->added = true;
    return BTM_OK;
}

int btm_mc_bind(btm_mc *h, void **local_ptr, void **mc_ptr)
{
    if (!h || !local_ptr || !mc_ptr) return set_error(BTM_ERR_INVALID, "multicast memory: null argument");
    if (!h->have_mc || !h->added || h->bound) return set_error(BTM_ERR_INVALID, "multicast memory: handle is not in a state to bind");
    if (!device_state(h->device)) return BTM_ERR_CUDA;
    int rc = BTM_OK;
    CUmemAllocationProp ap;
    memset(&ap, 0, sizeof(ap));
    ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    ap.location.id = h->device;
    ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    rc = check_cu(g_drv.MemCreate(&h->mem, h->bytes, &ap, 0), "cuMemCreate");
    if (rc) return rc;
    h->have_mem = true;
    // Would block until every rank of the team has added its device; the caller has made sure that all have.
    rc = check_cu(g_drv.MulticastBindMem(h->mc, 0, h->mem, 0, h->bytes, 0), "cuMulticastBindMem");
    if (rc) return rc;
    h->bound = true;
    CUmemAccessDesc ad;
    memset(&ad, 0, sizeof(ad));
    ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    ad.location.id = h->device;
    ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    rc = check_cu(g_drv.MemAddressReserve(&h->va_local, h->bytes, 0, 0, 0), "cuMemAddressReserve(local)");
    if (rc) return rc;
    rc = check_cu(g_drv.MemMap(h->va_local, h->bytes, 0, h->mem, 0), "cuMemMap(local)");
    if (rc) return rc;
    h->mapped_local = true;
    rc = check_cu(g_drv.MemSetAccess(h->va_local, h->bytes, &ad, 1), "cuMemSetAccess(local)");
    if (rc) return rc;
    rc = check_cu(g_drv.MemAddressReserve(&h->va_mc, h->bytes, 0, 0, 0), "cuMemAddressReserve(multicast)");
    if (rc) return rc;
    rc = check_cu(g_drv.MemMap(h->va_mc, h->bytes, 0, h->mc, 0), "cuMemMap(multicast)");
    if (rc) return rc;
    h->mapped_mc = true;
    rc = check_cu(g_drv.MemSetAccess(h->va_mc, h->bytes, &ad, 1), "cuMemSetAccess(multicast)");
    if (rc) return rc;
    *local_ptr = (void *)h->va_local;
    *mc_ptr = (void *)h->va_mc;
    return BTM_OK;
}

int btm_mc_release(btm_mc *h)
{
    if (!h) return BTM_OK;
    int first = BTM_OK;
    auto keep = [&](int rc) { if (rc && !first) first = rc; };
    if (g_drv.ready) {
        (void)cudaSetDevice(h->device);
        (void)cudaDeviceSynchronize(); // nothing of this device may still be storing through the mappings
        if (h->mapped_mc) keep(check_cu(g_drv.MemUnmap(h->va_mc, h->bytes), "cuMemUnmap(multicast)"));
        if (h->va_mc) keep(check_cu(g_drv.MemAddressFree(h->va_mc, h->bytes), "cuMemAddressFree(multicast)"));
        if (h->bound) keep(check_cu(g_drv.MulticastUnbind(h->mc, h->cu_dev, 0, h->bytes), "cuMulticastUnbind"));
        if (h->mapped_local) keep(check_cu(g_drv.MemUnmap(h->va_local, h->bytes), "cuMemUnmap(local)"));
        if (h->va_local) keep(check_cu(g_drv.MemAddressFree(h->va_local, h->bytes), "cuMemAddressFree(local)"));
        if (h->have_mem) keep(check_cu(g_drv.MemRelease(h->mem), "cuMemRelease(local)"));
        if (h->have_mc) keep(check_cu(g_drv.MemRelease(h->mc), "cuMemRelease(multicast)"));
    }
    delete h;
    return first;
}

} // extern "C"
