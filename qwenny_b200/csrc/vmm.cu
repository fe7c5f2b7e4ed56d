// Device memory mapped on demand (the reference's src/cuda/vmm.rs): a region reserves a range of device addresses once
// and maps physical pages into it only where data lives; the pages come from a pool shared by all regions, within a
// budget. Kernels and CUDA graphs see fixed addresses, so a slot's part of a cache costs memory only for the positions
// it holds, and a cache pool can be sized for the whole 180 GB part without committing it up front.
//
// Host code over the driver's virtual-memory calls. Unlike the reference, reads and writes through a region refuse
// ranges that are not mapped (there a copy from pages not mapped ends the process in the driver).
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

#include "../../include/qwenny_b200.h"

struct qb_pool {
    size_t page = 0;
    int dev = 0;
    std::mutex mu;
    std::vector<CUmemGenericAllocationHandle> free;
    size_t made = 0, budget = (size_t)-1;
};

struct qb_region {
    CUdeviceptr base = 0;
    size_t size = 0;
    std::vector<CUmemGenericAllocationHandle> pages;  // per page: its physical page, 0 when not mapped
    std::vector<char> mapped;
    qb_pool* pool = nullptr;
};

namespace {

// The driver's virtual-memory calls, resolved through the runtime when first needed: the library carries no link-time
// dependency on the driver, so it loads (and its host-side entries work) on a machine without one.
struct Drv {
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    bool ok = false;
};

const Drv* drv() {
    static Drv d;
    static bool tried = false;
    if (!tried) {
        tried = true;
        bool ok = true;
        auto get = [&](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult qr;
            if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess ||
                !*fn)
                ok = false;
        };
        get("cuMemGetAllocationGranularity", (void**)&d.MemGetAllocationGranularity);
        get("cuMemCreate", (void**)&d.MemCreate);
        get("cuMemRelease", (void**)&d.MemRelease);
        get("cuMemAddressReserve", (void**)&d.MemAddressReserve);
        get("cuMemAddressFree", (void**)&d.MemAddressFree);
        get("cuMemMap", (void**)&d.MemMap);
        get("cuMemUnmap", (void**)&d.MemUnmap);
        get("cuMemSetAccess", (void**)&d.MemSetAccess);
        d.ok = ok;
    }
    return d.ok ? &d : nullptr;
}

#define QB_DRV(x)                            \
    do {                                     \
        CUresult r_ = (x);                   \
        if (r_ != CUDA_SUCCESS) return 2000 + (int)r_; \
    } while (0)

CUmemAllocationProp prop_of(int dev) {
    CUmemAllocationProp p = {};
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = dev;
    return p;
}

// a new page from the driver; *h = 0 when the device has no more, which lowers the budget to the pages made
int create_page(qb_pool* p, CUmemGenericAllocationHandle* h) {
    *h = 0;
    const CUmemAllocationProp pr = prop_of(p->dev);
    CUresult r = drv()->MemCreate(h, p->page, &pr, 0);
    if (r == CUDA_ERROR_OUT_OF_MEMORY) {
        p->budget = p->made;
        *h = 0;
        return QB_OK;
    }
    QB_DRV(r);
    p->made++;
    return QB_OK;
}

int take_page(qb_pool* p, CUmemGenericAllocationHandle* h) {
    std::lock_guard<std::mutex> g(p->mu);
    *h = 0;
    if (!p->free.empty()) {
        *h = p->free.back();
        p->free.pop_back();
        return QB_OK;
    }
    if (p->made >= p->budget) return QB_OK;
    return create_page(p, h);
}

size_t available(qb_pool* p) {
    std::lock_guard<std::mutex> g(p->mu);
    return p->free.size() + (p->budget > p->made ? p->budget - p->made : 0);
}

bool all_mapped(const qb_region* r, size_t from, size_t n) {
    if (n == 0) return true;
    for (size_t i = from / r->pool->page; i <= (from + n - 1) / r->pool->page; i++)
        if (!r->mapped[i]) return false;
    return true;
}

}  // namespace

extern "C" {

// Pool::new: the page size is the device's minimum allocation granularity (2 MiB on current GPUs)
int qb_pool_create(int device, qb_pool** out) {
    if (!out) return QB_ERR_ARG;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaFree(0);  // the primary context, current on this thread for the driver calls below
    if (e != cudaSuccess) return (int)e;
    const Drv* D = drv();
    if (!D) return QB_ERR_UNSUPPORTED;
    qb_pool* p = new qb_pool();
    p->dev = device;
    const CUmemAllocationProp pr = prop_of(device);
    CUresult r = D->MemGetAllocationGranularity(&p->page, &pr, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
    if (r != CUDA_SUCCESS || p->page == 0) {
        delete p;
        return 2000 + (int)r;
    }
    *out = p;
    return QB_OK;
}

// (every region of the pool must have been freed)
void qb_pool_destroy(qb_pool* p) {
    if (!p) return;
    for (auto h : p->free) drv()->MemRelease(h);
    delete p;
}

size_t qb_pool_page(const qb_pool* p) { return p ? p->page : 0; }

// at most `pages` pages (those made already stay)
int qb_pool_set_budget(qb_pool* p, size_t pages) {
    if (!p) return QB_ERR_ARG;
    std::lock_guard<std::mutex> g(p->mu);
    p->budget = pages;
    return QB_OK;
}

// make the budget's pages now: the regions own that memory from the start (Pool::fill)
int qb_pool_fill(qb_pool* p) {
    if (!p) return QB_ERR_ARG;
    std::lock_guard<std::mutex> g(p->mu);
    while (p->made < p->budget) {
        CUmemGenericAllocationHandle h = 0;
        int rc = create_page(p, &h);
        if (rc) return rc;
        if (!h) break;
        p->free.push_back(h);
    }
    return QB_OK;
}

// give up to n free pages back to the driver, the budget lowered by as many (Pool::release)
int qb_pool_release(qb_pool* p, size_t n, size_t* given) {
    if (!p) return QB_ERR_ARG;
    std::lock_guard<std::mutex> g(p->mu);
    size_t k = n < p->free.size() ? n : p->free.size();
    for (size_t i = 0; i < k; i++) {
        QB_DRV(drv()->MemRelease(p->free.back()));
        p->free.pop_back();
        p->made--;
        p->budget--;
    }
    if (given) *given = k;
    return QB_OK;
}

// pages in use (mapped) and the budget
int qb_pool_usage(qb_pool* p, size_t* used, size_t* budget) {
    if (!p || !used || !budget) return QB_ERR_ARG;
    std::lock_guard<std::mutex> g(p->mu);
    *used = p->made - p->free.size();
    *budget = p->budget;
    return QB_OK;
}

size_t qb_pool_available(qb_pool* p) { return p ? available(p) : 0; }

// Region::reserve: `size` bytes of addresses (rounded up to whole pages); nothing is mapped yet
int qb_region_reserve(qb_pool* p, size_t size, qb_region** out) {
    if (!p || !out || size == 0) return QB_ERR_ARG;
    cudaError_t e = cudaSetDevice(p->dev);
    if (e != cudaSuccess) return (int)e;
    qb_region* r = new qb_region();
    r->pool = p;
    r->size = (size + p->page - 1) / p->page * p->page;
    CUresult rc = drv()->MemAddressReserve(&r->base, r->size, p->page, 0, 0);
    if (rc != CUDA_SUCCESS) {
        delete r;
        return 2000 + (int)rc;
    }
    r->pages.assign(r->size / p->page, 0);
    r->mapped.assign(r->size / p->page, 0);
    *out = r;
    return QB_OK;
}

void* qb_region_ptr(const qb_region* r) { return r ? (void*)r->base : nullptr; }
size_t qb_region_size(const qb_region* r) { return r ? r->size : 0; }
int qb_region_is_mapped(const qb_region* r, size_t from, size_t to) {
    return r && from <= to && to <= r->size && all_mapped(r, from, to - from);
}

// Region::map: the pages covering bytes [from, to), zeroed on `stream`; *ok = 0 (and nothing more mapped) when the
// pool has too few
int qb_region_map(qb_region* r, void* stream, size_t from, size_t to, int* ok) {
    if (!r || !ok || from > to) return QB_ERR_ARG;
    qb_pool* p = r->pool;
    if (to > r->size) to = r->size;
    const size_t p0 = from / p->page, p1 = (to + p->page - 1) / p->page;
    size_t need = 0;
    for (size_t i = p0; i < p1; i++) need += !r->mapped[i];
    *ok = 1;
    if (need == 0) return QB_OK;
    if (available(p) < need) {
        *ok = 0;
        return QB_OK;
    }
    CUmemAccessDesc access = {};
    access.location = prop_of(p->dev).location;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (size_t i = p0; i < p1; i++) {
        if (r->mapped[i]) continue;
        CUmemGenericAllocationHandle h = 0;
        int rc = take_page(p, &h);
        if (rc) return rc;
        if (!h) return QB_ERR_TOO_LARGE;  // another region took the pages in between
        const CUdeviceptr at = r->base + i * p->page;
        // (a page the driver refuses to map goes back to the pool: nothing is lost on the way out)
        CUresult mr = drv()->MemMap(at, p->page, 0, h, 0);
        if (mr == CUDA_SUCCESS) {
            mr = drv()->MemSetAccess(at, p->page, &access, 1);
            if (mr != CUDA_SUCCESS) drv()->MemUnmap(at, p->page);
        }
        if (mr != CUDA_SUCCESS) {
            std::lock_guard<std::mutex> g(p->mu);
            p->free.push_back(h);
            return 2000 + (int)mr;
        }
        r->pages[i] = h;
        r->mapped[i] = 1;
        {
            cudaError_t e = cudaMemsetAsync((void*)at, 0, p->page, (cudaStream_t)stream);
            if (e != cudaSuccess) return (int)e;
        }
    }
    return QB_OK;
}

// Region::unmap: the pages that lie wholly inside bytes [from, to), after the stream's work on them
int qb_region_unmap(qb_region* r, void* stream, size_t from, size_t to) {
    if (!r || from > to) return QB_ERR_ARG;
    qb_pool* p = r->pool;
    if (to > r->size) to = r->size;
    const size_t p0 = (from + p->page - 1) / p->page, p1 = to / p->page;
    bool any = false;
    for (size_t i = p0; i < p1; i++) any |= r->mapped[i] != 0;
    if (!any) return QB_OK;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    for (size_t i = p0; i < p1; i++) {
        if (!r->mapped[i]) continue;
        QB_DRV(drv()->MemUnmap(r->base + i * p->page, p->page));
        std::lock_guard<std::mutex> g(p->mu);
        p->free.push_back(r->pages[i]);
        r->pages[i] = 0;
        r->mapped[i] = 0;
    }
    return QB_OK;
}

// Region::read / write: bytes [from, from + n) to / from the host; the range must be mapped (QB_ERR_ARG otherwise)
int qb_region_read(qb_region* r, void* stream, size_t from, void* out, size_t n) {
    if (!r || !out || from + n < from || from + n > r->size || !all_mapped(r, from, n)) return QB_ERR_ARG;
    if (n == 0) return QB_OK;
    cudaError_t e = cudaMemcpyAsync(out, (const void*)(r->base + from), n, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    return e == cudaSuccess ? QB_OK : (int)e;
}

int qb_region_write(qb_region* r, void* stream, size_t from, const void* data, size_t n) {
    if (!r || !data || from + n < from || from + n > r->size || !all_mapped(r, from, n)) return QB_ERR_ARG;
    if (n == 0) return QB_OK;
    // on the stream, waited for: the stream's next kernels would not wait for a copy on the legacy stream
    cudaError_t e = cudaMemcpyAsync((void*)(r->base + from), data, n, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    return e == cudaSuccess ? QB_OK : (int)e;
}

// unmaps what is mapped (after the stream's work), gives the pages back to the pool and frees the addresses
int qb_region_free(qb_region* r, void* stream) {
    if (!r) return QB_OK;
    int rc = qb_region_unmap(r, stream, 0, r->size);
    CUresult f = drv()->MemAddressFree(r->base, r->size);
    delete r;
    return rc ? rc : (f == CUDA_SUCCESS ? QB_OK : 2000 + (int)f);
}

}  // extern "C"
