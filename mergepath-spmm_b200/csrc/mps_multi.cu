// Single-process multi-GPU driver (no reference counterpart: the reference is single-GPU).
//
// A is cut into contiguous row slabs of equal (nnz + 4*rows), slab g lives on device g together with a
// full copy of B; every device multiplies its slab into its own place of a full-height C buffer, so no
// exchange is needed for the multiply.  A replicated C, when asked for, is one grouped NCCL broadcast
// per slab (unequal slab heights) over NVLink.  One host thread drives all devices: every call below is
// asynchronous per device except where it says it waits.  NCCL is looked up with dlopen at the first
// gather, so the library loads and the multiply works on machines without it.
#include "mps.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

#include "mps_internal.h"

using mps::fail;

namespace {

#define MM_CUDA(call)                                                                                \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess) return fail(MPS_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));  \
    } while (0)

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool load() {
        if (handle) return true;
        handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!handle) handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!handle) return false;
        CommInitAll = (decltype(CommInitAll))dlsym(handle, "ncclCommInitAll");
        CommDestroy = (decltype(CommDestroy))dlsym(handle, "ncclCommDestroy");
        GroupStart = (decltype(GroupStart))dlsym(handle, "ncclGroupStart");
        GroupEnd = (decltype(GroupEnd))dlsym(handle, "ncclGroupEnd");
        Broadcast = (decltype(Broadcast))dlsym(handle, "ncclBroadcast");
        AllGather = (decltype(AllGather))dlsym(handle, "ncclAllGather");
        GetErrorString = (decltype(GetErrorString))dlsym(handle, "ncclGetErrorString");
        return CommInitAll && CommDestroy && GroupStart && GroupEnd && Broadcast && AllGather && GetErrorString;
    }
};
NcclApi g_nccl;

struct Slab {
    int device = 0, row0 = 0, row1 = 0, nnz = 0;
    int32_t *d_rp = nullptr, *d_col = nullptr;
    void *d_val = nullptr, *d_B = nullptr, *d_C = nullptr;  // d_C: full height, n_rows x dim
    mps_plan *plan = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

}  // namespace

struct mps_multi {
    int n_gpus = 0, n_rows = 0, n_cols = 0, nnz = 0, dim = 0, dtype = 0;
    bool has_val = false, have_b = false;
    bool distinct = true;     // every slab on a device of its own (what a communicator needs)
    size_t b_block_rows = 0;  // rows of B per device block: ceil(n_cols / n_gpus); every d_B holds n_gpus such blocks
    std::vector<Slab> slab;
    std::vector<ncclComm_t> comm;  // empty until the first gather
};

static size_t elem_bytes(int dtype) { return dtype == MPS_F16 ? 2 : 4; }

extern "C" void mps_multi_destroy(mps_multi *m) {
    if (!m) return;
    for (size_t g = 0; g < m->comm.size(); ++g)
        if (m->comm[g] && g_nccl.CommDestroy) g_nccl.CommDestroy(m->comm[g]);
    for (Slab &s : m->slab) {
        cudaSetDevice(s.device);
        mps_plan_destroy(s.plan);
        cudaFree(s.d_rp); cudaFree(s.d_col); cudaFree(s.d_val); cudaFree(s.d_B); cudaFree(s.d_C);
        if (s.ev0) cudaEventDestroy(s.ev0);
        if (s.ev1) cudaEventDestroy(s.ev1);
        if (s.stream) cudaStreamDestroy(s.stream);
    }
    delete m;
}

extern "C" int mps_multi_create(int32_t n_gpus, const int32_t *devices, int32_t n_rows, int32_t n_cols, int32_t dim, int dtype,
                                int32_t cost, int32_t threads_per_warp, const int32_t *row_ptr, const int32_t *col_idx, const void *val,
                                mps_multi **out) {
    if (!out) return fail(MPS_ERR_ARG, "mps_multi_create: out is NULL");
    *out = nullptr;
    if (n_gpus < 1 || n_gpus > 64 || !row_ptr || n_rows < 0 || n_cols < 0 || dim < 1 || cost < 1)
        return fail(MPS_ERR_ARG, "mps_multi_create: bad argument");
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "mps_multi_create: unknown dtype %d", dtype);
    if (row_ptr[n_rows] < 0 || (row_ptr[n_rows] > 0 && !col_idx)) return fail(MPS_ERR_ARG, "mps_multi_create: bad nnz / col_idx");
    if ((long long)n_rows + 1 + row_ptr[n_rows] >= 1ll << 31) return fail(MPS_ERR_UNSUPPORTED, "mps_multi_create: N+1+nnz does not fit 31 bits");
    // the caller's arrays are checked on the host before anything is uploaded: a bad index must not become a gather
    // outside B on some device
    if (int rc = mps::check_csr_host("mps_multi_create", n_rows, n_cols, row_ptr, col_idx, 0)) return rc;
    int visible = 0;
    MM_CUDA(cudaGetDeviceCount(&visible));
    for (int g = 0; g < n_gpus; ++g) {
        const int d = devices ? devices[g] : g;
        if (d < 0 || d >= visible) return fail(MPS_ERR_ARG, "mps_multi_create: device %d of %d requested, %d visible", d, n_gpus, visible);
    }
    const int nnz = row_ptr[n_rows];
    mps_multi *m = new (std::nothrow) mps_multi();
    if (!m) return fail(MPS_ERR_NOMEM, "mps_multi_create: out of host memory");
    m->n_gpus = n_gpus; m->n_rows = n_rows; m->n_cols = n_cols; m->nnz = nnz; m->dim = dim; m->dtype = dtype; m->has_val = val != nullptr;
    m->slab.resize((size_t)n_gpus);
    m->b_block_rows = ((size_t)n_cols + (size_t)n_gpus - 1) / (size_t)n_gpus;
    for (int g = 0; g < n_gpus; ++g)
        for (int h = 0; h < g; ++h)
            if ((devices ? devices[g] : g) == (devices ? devices[h] : h)) m->distinct = false;
    std::vector<int32_t> bounds((size_t)n_gpus + 1);
    int rc = mps_slab_bounds_items(row_ptr, n_rows, n_gpus, 4, bounds.data());
    const size_t es = elem_bytes(dtype);
    int prev = 0;
    cudaGetDevice(&prev);
    for (int g = 0; g < n_gpus && rc == MPS_OK; ++g) {
        Slab &s = m->slab[(size_t)g];
        s.device = devices ? devices[g] : g;
        s.row0 = bounds[(size_t)g]; s.row1 = bounds[(size_t)g + 1];
        const int rows = s.row1 - s.row0, k0 = row_ptr[s.row0];
        s.nnz = row_ptr[s.row1] - k0;
        std::vector<int32_t> rp((size_t)rows + 1);
        rc = mps_slab_rebase(row_ptr, s.row0, s.row1, rp.data());
        if (rc != MPS_OK) break;
        cudaError_t e = cudaSetDevice(s.device);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreate(&s.ev0);
        if (e == cudaSuccess) e = cudaEventCreate(&s.ev1);
        if (e == cudaSuccess) e = cudaMalloc(&s.d_rp, 4 * ((size_t)rows + 1));
        if (e == cudaSuccess) e = cudaMalloc(&s.d_col, 4 * (size_t)(s.nnz ? s.nnz : 4));
        if (e == cudaSuccess && val) e = cudaMalloc(&s.d_val, es * (size_t)(s.nnz ? s.nnz : 8));
        if (e == cudaSuccess) e = cudaMalloc(&s.d_B, es * m->b_block_rows * (size_t)n_gpus * dim + 16);
        if (e == cudaSuccess) e = cudaMalloc(&s.d_C, es * (size_t)n_rows * dim + 16);
        if (e == cudaSuccess) e = cudaMemcpy(s.d_rp, rp.data(), 4 * ((size_t)rows + 1), cudaMemcpyHostToDevice);
        if (e == cudaSuccess && s.nnz) e = cudaMemcpy(s.d_col, col_idx + k0, 4 * (size_t)s.nnz, cudaMemcpyHostToDevice);
        if (e == cudaSuccess && val && s.nnz) e = cudaMemcpy(s.d_val, (const char *)val + es * (size_t)k0, es * (size_t)s.nnz, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { rc = fail(MPS_ERR_CUDA, "mps_multi_create: device %d: %s", s.device, cudaGetErrorString(e)); break; }
        rc = mps_plan_create(rows, s.nnz, dim, dtype, cost, threads_per_warp, &s.plan);
        if (rc == MPS_OK) rc = mps_plan_partition(s.plan, s.d_rp, s.stream);
    }
    cudaSetDevice(prev);
    if (rc != MPS_OK) { mps_multi_destroy(m); return rc; }
    *out = m;
    return MPS_OK;
}

extern "C" int mps_multi_slab(const mps_multi *m, int32_t g, int32_t *device, int32_t *row0, int32_t *row1, int32_t *nnz, void **d_C) {
    if (!m || g < 0 || g >= m->n_gpus) return fail(MPS_ERR_ARG, "mps_multi_slab: bad argument");
    const Slab &s = m->slab[(size_t)g];
    if (device) *device = s.device;
    if (row0) *row0 = s.row0;
    if (row1) *row1 = s.row1;
    if (nnz) *nnz = s.nnz;
    if (d_C) *d_C = s.d_C;
    return MPS_OK;
}

// Communicators are created once, outside any timed region.
static int multi_init_comm(mps_multi *m) {
    if (m->n_gpus > 1 && m->comm.empty()) {
        if (!m->distinct) return fail(MPS_ERR_UNSUPPORTED, "a communicator needs every slab on a device of its own");
        if (!g_nccl.load()) return fail(MPS_ERR_UNSUPPORTED, "NCCL is needed (libnccl.so.2 not found: %s)", dlerror());
        std::vector<int> devs;
        for (const Slab &s : m->slab) devs.push_back(s.device);
        m->comm.assign((size_t)m->n_gpus, nullptr);
        ncclResult_t r = g_nccl.CommInitAll(m->comm.data(), m->n_gpus, devs.data());
        if (r != ncclSuccess) { m->comm.clear(); return fail(MPS_ERR_CUDA, "ncclCommInitAll: %s", g_nccl.GetErrorString(r)); }
    }
    return MPS_OK;
}

// B reaches every device once over PCIe in total, not once per device: device g uploads block g of B's rows
// (ceil(n_cols / n_gpus) rows each) into its place of its own full-size buffer, then one in-place NCCL
// all-gather of equal blocks over NVLink completes every copy.  Without NCCL, with one device, or with several
// slabs on one device (no communicator possible) every device uploads all of B itself.
extern "C" int mps_multi_set_b(mps_multi *m, const void *host_B) {
    if (!m || !host_B) return fail(MPS_ERR_ARG, "mps_multi_set_b: NULL argument");
    const size_t es = elem_bytes(m->dtype), row_bytes = es * (size_t)m->dim;
    int prev = 0;
    cudaGetDevice(&prev);
    bool over_nvlink = m->n_gpus > 1 && m->distinct && multi_init_comm(m) == MPS_OK;
    int rc = MPS_OK;
    for (int g = 0; g < m->n_gpus && rc == MPS_OK; ++g) {
        Slab &s = m->slab[(size_t)g];
        size_t row0 = 0, rows = (size_t)m->n_cols;
        if (over_nvlink) {
            row0 = std::min((size_t)g * m->b_block_rows, (size_t)m->n_cols);
            rows = std::min(m->b_block_rows, (size_t)m->n_cols - row0);
        }
        cudaError_t e = cudaSetDevice(s.device);
        if (e == cudaSuccess && rows)
            e = cudaMemcpyAsync((char *)s.d_B + row0 * row_bytes, (const char *)host_B + row0 * row_bytes, rows * row_bytes, cudaMemcpyHostToDevice, s.stream);
        if (e != cudaSuccess) rc = fail(MPS_ERR_CUDA, "mps_multi_set_b: device %d: %s", s.device, cudaGetErrorString(e));
    }
    if (rc == MPS_OK && over_nvlink) {
        const size_t count = m->b_block_rows * (size_t)m->dim;
        const ncclDataType_t dt = m->dtype == MPS_F16 ? ncclFloat16 : ncclFloat32;
        ncclResult_t r = g_nccl.GroupStart();
        for (int g = 0; g < m->n_gpus && r == ncclSuccess; ++g) {
            Slab &s = m->slab[(size_t)g];
            r = g_nccl.AllGather((const char *)s.d_B + (size_t)g * count * es, s.d_B, count, dt, m->comm[(size_t)g], s.stream);
        }
        ncclResult_t r2 = g_nccl.GroupEnd();
        if (r != ncclSuccess || r2 != ncclSuccess) rc = fail(MPS_ERR_CUDA, "ncclAllGather: %s", g_nccl.GetErrorString(r != ncclSuccess ? r : r2));
    }
    for (Slab &s : m->slab) {  // drain every device, also after a failure: the caller may free host_B next
        cudaSetDevice(s.device);
        cudaError_t e = cudaStreamSynchronize(s.stream);
        if (e != cudaSuccess && rc == MPS_OK) rc = fail(MPS_ERR_CUDA, "mps_multi_set_b: device %d: %s", s.device, cudaGetErrorString(e));
    }
    cudaSetDevice(prev);
    if (rc == MPS_OK) m->have_b = true;
    return rc;
}

static int multi_gather(mps_multi *m) {
    if (m->n_gpus == 1) return MPS_OK;
    const size_t es = elem_bytes(m->dtype);
    const ncclDataType_t dt = m->dtype == MPS_F16 ? ncclFloat16 : ncclFloat32;
    ncclResult_t r = g_nccl.GroupStart();
    for (int root = 0; root < m->n_gpus && r == ncclSuccess; ++root) {
        const Slab &src = m->slab[(size_t)root];
        const size_t count = (size_t)(src.row1 - src.row0) * m->dim, at = es * (size_t)src.row0 * m->dim;
        if (!count) continue;
        for (int g = 0; g < m->n_gpus && r == ncclSuccess; ++g) {
            Slab &s = m->slab[(size_t)g];
            r = g_nccl.Broadcast((const char *)s.d_C + at, (char *)s.d_C + at, count, dt, root, m->comm[(size_t)g], s.stream);
        }
    }
    ncclResult_t r2 = g_nccl.GroupEnd();
    if (r != ncclSuccess || r2 != ncclSuccess) return fail(MPS_ERR_CUDA, "ncclBroadcast: %s", g_nccl.GetErrorString(r != ncclSuccess ? r : r2));
    return MPS_OK;
}

extern "C" int mps_multi_spmm(mps_multi *m, int32_t repeat, int32_t gather_c, float *ms_spmm, float *ms_gather) {
    if (!m || repeat < 1) return fail(MPS_ERR_ARG, "mps_multi_spmm: bad argument");
    if (!m->have_b) return fail(MPS_ERR_STATE, "mps_multi_spmm: call mps_multi_set_b first");
    const size_t es = elem_bytes(m->dtype);
    int prev = 0;
    cudaGetDevice(&prev);
    int rc = MPS_OK;
    for (Slab &s : m->slab) {  // start marks on every device, then launches: all devices run at once
        cudaSetDevice(s.device);
        cudaEventRecord(s.ev0, s.stream);
    }
    for (int i = 0; i < repeat && rc == MPS_OK; ++i)
        for (Slab &s : m->slab) {
            cudaSetDevice(s.device);
            rc = mps_spmm(s.plan, s.d_rp, s.d_col, s.d_val, s.d_B, (char *)s.d_C + es * (size_t)s.row0 * m->dim, s.stream);
            if (rc != MPS_OK) break;
        }
    float worst = 0.0f;
    for (Slab &s : m->slab) {
        cudaSetDevice(s.device);
        cudaEventRecord(s.ev1, s.stream);
    }
    for (Slab &s : m->slab) {  // every device is drained, also after a failed launch: nothing of this call stays in flight
        cudaSetDevice(s.device);
        if (rc == MPS_OK) rc = mps_plan_sync_check(s.plan, s.stream);
        else cudaStreamSynchronize(s.stream);
        float ms = 0.0f;
        if (rc == MPS_OK && cudaEventElapsedTime(&ms, s.ev0, s.ev1) == cudaSuccess && ms > worst) worst = ms;
    }
    if (ms_spmm) *ms_spmm = worst / repeat;
    if (rc == MPS_OK && gather_c) rc = multi_init_comm(m);
    if (rc == MPS_OK && gather_c) {
        for (Slab &s : m->slab) { cudaSetDevice(s.device); cudaEventRecord(s.ev0, s.stream); }
        rc = multi_gather(m);
        float worst_g = 0.0f;
        for (Slab &s : m->slab) { cudaSetDevice(s.device); cudaEventRecord(s.ev1, s.stream); }
        for (Slab &s : m->slab) {
            cudaSetDevice(s.device);
            cudaError_t e = cudaStreamSynchronize(s.stream);
            if (e != cudaSuccess && rc == MPS_OK) rc = fail(MPS_ERR_CUDA, "mps_multi_spmm: gather on device %d: %s", s.device, cudaGetErrorString(e));
            float ms = 0.0f;
            if (rc == MPS_OK && cudaEventElapsedTime(&ms, s.ev0, s.ev1) == cudaSuccess && ms > worst_g) worst_g = ms;
        }
        if (ms_gather) *ms_gather = worst_g;
    } else if (ms_gather) {
        *ms_gather = 0.0f;
    }
    cudaSetDevice(prev);
    return rc;
}

extern "C" int mps_multi_get_c(mps_multi *m, void *host_C, int32_t from_gpu) {
    if (!m || !host_C || from_gpu >= m->n_gpus) return fail(MPS_ERR_ARG, "mps_multi_get_c: bad argument");
    const size_t es = elem_bytes(m->dtype);
    int prev = 0;
    cudaGetDevice(&prev);
    int rc = MPS_OK;
    if (from_gpu >= 0) {  // the whole C as device `from_gpu` holds it (meaningful after a gather)
        Slab &s = m->slab[(size_t)from_gpu];
        cudaSetDevice(s.device);
        cudaError_t e = cudaMemcpy(host_C, s.d_C, es * (size_t)m->n_rows * m->dim, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) rc = fail(MPS_ERR_CUDA, "mps_multi_get_c: %s", cudaGetErrorString(e));
    } else {  // every slab from the device that computed it
        for (Slab &s : m->slab) {
            cudaSetDevice(s.device);
            const size_t at = es * (size_t)s.row0 * m->dim, bytes = es * (size_t)(s.row1 - s.row0) * m->dim;
            cudaError_t e = bytes ? cudaMemcpy((char *)host_C + at, (char *)s.d_C + at, bytes, cudaMemcpyDeviceToHost) : cudaSuccess;
            if (e != cudaSuccess) { rc = fail(MPS_ERR_CUDA, "mps_multi_get_c: device %d: %s", s.device, cudaGetErrorString(e)); break; }
        }
    }
    cudaSetDevice(prev);
    return rc;
}
