// MergePathSpMM <input_file> <dimension> <cost> <threads_per_warp> <repeat> [--key=value ...]
//
// Command-line twin of the reference program (src/MergePathSpMM.cu:110-277; fp16: the same argv in
// src/MergePathSpMM_fp16.cu:111-278): same five positionals in the same order, same usage text and
// exit status when fewer are given (:114-117), same first output line (:141).  After that line it
// prints what the reference leaves to an external profiler: time per SpMM, GFLOP/s = 2*nnz*dim/t,
// algorithmic GB/s.  B is filled with ones as in the reference (:180-182); A's values are all ones
// (the file has none) unless --values=gcn.
//
// Options (all optional, after the positionals):
//   --dtype=f32|f16   --values=unit|gcn   --check   --device=K
//   --gpus=G          row slabs of equal (nnz + 4*rows) over G devices of this node, one host thread per device
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <thread>
#include <vector>

#include "mps.h"

namespace {

struct Options {
    std::string dtype = "f32", values = "unit";
    bool check = false;
    int device = 0, gpus = 1;
};

bool parse_option(const char *arg, Options &o) {
    std::string a(arg);
    auto val = [&](const char *key) -> const char * {
        size_t n = strlen(key);
        return a.compare(0, n, key) == 0 ? arg + n : nullptr;
    };
    if (const char *v = val("--dtype=")) { o.dtype = v; return o.dtype == "f32" || o.dtype == "f16"; }
    if (const char *v = val("--values=")) { o.values = v; return o.values == "unit" || o.values == "gcn"; }
    if (const char *v = val("--device=")) { o.device = atoi(v); return true; }
    if (const char *v = val("--gpus=")) { o.gpus = atoi(v); return o.gpus >= 1; }
    if (a == "--check") { o.check = true; return true; }
    return false;
}

#define CUDA_OK(call)                                                                      \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            fprintf(stderr, "CUDA error: %s (%s)\n", cudaGetErrorString(e_), #call);       \
            return 1;                                                                      \
        }                                                                                  \
    } while (0)
#define MPS_OK_OR_DIE(call)                                              \
    do {                                                                 \
        if ((call) != MPS_OK) {                                          \
            fprintf(stderr, "error: %s\n", mps_last_error());            \
            return 1;                                                    \
        }                                                                \
    } while (0)

struct SlabResult {
    double ms_per_spmm = 0, partition_ms = 0;
    int rc = 0;
    long long bad = 0;
};

// One device: upload the slab [row0,row1) and all of B, partition, warm up, time `repeat` launches.
int run_slab(const mps_csr &g, const std::vector<float> &val, int row0, int row1, int dim, int cost, int tpw, int repeat,
             const Options &o, int device, SlabResult *out) {
    CUDA_OK(cudaSetDevice(device));
    const bool half = o.dtype == "f16";
    const int n = row1 - row0;
    const int k0 = g.row_ptr[row0], nnz = g.row_ptr[row1] - k0;
    const size_t es = half ? 2 : 4;
    std::vector<int32_t> rp((size_t)n + 1);
    MPS_OK_OR_DIE(mps_slab_rebase(g.row_ptr, row0, row1, rp.data()));

    int32_t *d_rp = nullptr, *d_col = nullptr;
    void *d_val = nullptr, *d_B = nullptr, *d_C = nullptr;
    CUDA_OK(cudaMalloc(&d_rp, 4 * ((size_t)n + 1)));
    CUDA_OK(cudaMalloc(&d_col, 4 * (size_t)(nnz ? nnz : 1)));
    CUDA_OK(cudaMalloc(&d_B, es * (size_t)g.n_rows * dim + 16));
    CUDA_OK(cudaMalloc(&d_C, es * (size_t)n * dim + 16));
    CUDA_OK(cudaMemcpy(d_rp, rp.data(), 4 * ((size_t)n + 1), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_col, g.col_idx + k0, 4 * (size_t)nnz, cudaMemcpyHostToDevice));
    if (!val.empty()) {
        CUDA_OK(cudaMalloc(&d_val, es * (size_t)(nnz ? nnz : 1)));
        if (half) {
            std::vector<__half> hv((size_t)nnz);
            for (int k = 0; k < nnz; ++k) hv[(size_t)k] = __float2half(val[(size_t)k0 + k]);
            CUDA_OK(cudaMemcpy(d_val, hv.data(), 2 * (size_t)nnz, cudaMemcpyHostToDevice));
        } else {
            CUDA_OK(cudaMemcpy(d_val, val.data() + k0, 4 * (size_t)nnz, cudaMemcpyHostToDevice));
        }
    }
    {   // B = 1 everywhere, as the reference fills it
        const size_t cells = (size_t)g.n_rows * dim;
        if (half) { std::vector<__half> b(cells, __float2half(1.0f)); CUDA_OK(cudaMemcpy(d_B, b.data(), 2 * cells, cudaMemcpyHostToDevice)); }
        else { std::vector<float> b(cells, 1.0f); CUDA_OK(cudaMemcpy(d_B, b.data(), 4 * cells, cudaMemcpyHostToDevice)); }
    }
    mps_plan *plan = nullptr;
    MPS_OK_OR_DIE(mps_plan_create(n, nnz, dim, half ? MPS_F16 : MPS_F32, cost, tpw, &plan));
    auto t0 = std::chrono::steady_clock::now();
    MPS_OK_OR_DIE(mps_plan_partition(plan, d_rp, nullptr));
    out->partition_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    for (int i = 0; i < 3; ++i) MPS_OK_OR_DIE(mps_spmm(plan, d_rp, d_col, d_val, d_B, d_C, nullptr));
    cudaEvent_t e0, e1;
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaEventRecord(e0));
    for (int i = 0; i < repeat; ++i) MPS_OK_OR_DIE(mps_spmm(plan, d_rp, d_col, d_val, d_B, d_C, nullptr));
    CUDA_OK(cudaEventRecord(e1));
    MPS_OK_OR_DIE(mps_plan_sync_check(plan, nullptr));
    float ms = 0;
    CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
    out->ms_per_spmm = repeat > 0 ? ms / repeat : 0.0;

    if (o.check) {  // with B == 1 every element of row i is the sum of the row's values
        std::vector<unsigned char> hc(es * (size_t)n * dim);
        CUDA_OK(cudaMemcpy(hc.data(), d_C, hc.size(), cudaMemcpyDeviceToHost));
        for (int i = 0; i < n; ++i) {
            double want = 0;
            for (int k = rp[(size_t)i]; k < rp[(size_t)i + 1]; ++k) want += val.empty() ? 1.0 : (half ? (double)__half2float(__float2half(val[(size_t)k0 + k])) : (double)val[(size_t)k0 + k]);
            const double tol = (half ? 1e-2 : 1e-5) * std::fabs(want) + 1e-6;
            for (int j = 0; j < dim; ++j) {
                const double got = half ? (double)__half2float(((const __half *)hc.data())[(size_t)i * dim + j]) : (double)((const float *)hc.data())[(size_t)i * dim + j];
                if (std::fabs(got - want) > tol) ++out->bad;
            }
        }
    }
    mps_plan_destroy(plan);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(d_rp); cudaFree(d_col); cudaFree(d_val); cudaFree(d_B); cudaFree(d_C);
    return 0;
}

}  // namespace

int main(int argc, char *argv[]) {
    if (argc < 6) {
        std::cout << "Usage: ./application <input_file> <dimension> <cost> <threads_per_warp> <repeat>" << std::endl;
        exit(-1);
    }
    const int dim = atoi(argv[2]), cost = atoi(argv[3]), tpw = atoi(argv[4]), repeat = atoi(argv[5]);
    Options o;
    for (int i = 6; i < argc; ++i)
        if (!parse_option(argv[i], o)) { fprintf(stderr, "unknown or malformed option %s\n", argv[i]); return 2; }

    mps_csr g;
    if (mps_csr_load(argv[1], 0, &g) != MPS_OK) { fprintf(stderr, "error: %s\n", mps_last_error()); return 1; }
    std::cout << "Total number of rows: " << g.n_rows << " and non-zeros: " << g.nnz << std::endl;
    if (dim < 1 || cost < 1) { fprintf(stderr, "error: dimension and cost must be >= 1\n"); return 2; }
    if (dim <= 32 && tpw > 32 / dim)
        fprintf(stderr, "note: threads_per_warp %d exceeds 32/dim = %d; using %d (the reference exits here)\n", tpw, 32 / dim, 32 / dim);

    std::vector<float> val;
    if (o.values == "gcn") {
        val.resize((size_t)g.nnz);
        for (int i = 0; i < g.n_rows; ++i) {
            const double di = g.row_ptr[i + 1] - g.row_ptr[i];
            for (int k = g.row_ptr[i]; k < g.row_ptr[i + 1]; ++k) {
                const int j = g.col_idx[k];
                const double dj = g.row_ptr[j + 1] - g.row_ptr[j];
                val[(size_t)k] = (float)(1.0 / std::sqrt(di * dj));
            }
        }
    }
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess || visible < 1) { fprintf(stderr, "error: no CUDA device\n"); return 1; }
    if (o.gpus > visible) { fprintf(stderr, "error: --gpus=%d but only %d devices are visible\n", o.gpus, visible); return 1; }

    std::vector<int32_t> bounds((size_t)o.gpus + 1);
    if (mps_slab_bounds_items(g.row_ptr, g.n_rows, o.gpus, /*row_weight=*/4, bounds.data()) != MPS_OK) { fprintf(stderr, "error: %s\n", mps_last_error()); return 1; }
    std::vector<SlabResult> res((size_t)o.gpus);
    std::vector<std::thread> th;
    for (int s = 0; s < o.gpus; ++s)
        th.emplace_back([&, s] {
            res[(size_t)s].rc = run_slab(g, val, bounds[(size_t)s], bounds[(size_t)s + 1], dim, cost, tpw, repeat, o,
                                         o.gpus == 1 ? o.device : s, &res[(size_t)s]);
        });
    for (auto &t : th) t.join();
    double ms = 0, part = 0;
    long long bad = 0;
    for (const SlabResult &r : res) {
        if (r.rc) return r.rc;
        if (r.ms_per_spmm > ms) ms = r.ms_per_spmm;
        if (r.partition_ms > part) part = r.partition_ms;
        bad += r.bad;
    }
    const double flops = 2.0 * g.nnz * dim;
    const double bytes = (double)mps_algorithmic_bytes(g.n_rows, g.nnz, dim, o.dtype == "f16" ? MPS_F16 : MPS_F32, o.values == "gcn");
    printf("gpus: %d  dtype: %s  values: %s  dim: %d  cost: %d  repeat: %d\n", o.gpus, o.dtype.c_str(), o.values.c_str(), dim, cost, repeat);
    printf("partition: %.3f ms (once)\n", part);
    if (repeat > 0)
        printf("time per SpMM: %.4f ms  %.1f GFLOP/s  %.1f GB/s algorithmic (max over devices)\n", ms, flops / ms / 1e6, bytes / ms / 1e6);
    if (o.check) printf("check: %lld elements outside tolerance\n", bad);
    mps_csr_free(&g);
    return bad ? 3 : 0;
}
