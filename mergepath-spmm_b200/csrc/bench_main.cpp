// MergePathSpMM <input_file> <dimension> <cost> <threads_per_warp> <repeat> [--key=value ...]
//
// Command-line twin of the reference program (src/MergePathSpMM.cu:110-277; fp16: the same argv in
// src/MergePathSpMM_fp16.cu:111-278): same five positionals in the same order, same usage text and
// exit status when fewer are given (:114-117), same first output line (:141).  After that line it
// prints what the reference leaves to an external profiler: time per SpMM, GFLOP/s = 2*nnz*dim/t,
// algorithmic GB/s.  B is filled with ones as in the reference (:180-182); A's values are all ones
// (the file has none) unless --values=gcn.
//
// Installed under a name that ends in "_fp16" (the build links MergePathSpMM_fp16 to the same program) it is the
// twin of the reference's fp16 program: the same argv, fp16 storage unless --dtype says otherwise.
//
// <input_file> may also be the binary sidecar that mps_csr_save_bin writes (a 10^9-edge graph is ~10 GB of text).
//
// Options (all optional, after the positionals):
//   --dtype=f32|f16   --values=unit|gcn   --check   --device=K
//   --gpus=G          row slabs of equal (nnz + 4*rows) over G devices of this node (mps_multi_*)
//   --gather-c        after the timed multiplies, replicate C on every device with NCCL and time it
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

#include "mps.h"

namespace {

struct Options {
    std::string dtype = "f32", values = "unit";
    bool check = false, gather_c = false;
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
    if (a == "--gather-c") { o.gather_c = true; return true; }
    return false;
}

#define MPS_OK_OR_DIE(call)                                              \
    do {                                                                 \
        if ((call) != MPS_OK) {                                          \
            fprintf(stderr, "error: %s\n", mps_last_error());            \
            return 1;                                                    \
        }                                                                \
    } while (0)

float half_to_float(uint16_t h) { return __half2float(*reinterpret_cast<const __half *>(&h)); }

}  // namespace

int main(int argc, char *argv[]) {
    if (argc < 6) {
        std::cout << "Usage: ./application <input_file> <dimension> <cost> <threads_per_warp> <repeat>" << std::endl;
        exit(-1);
    }
    const int dim = atoi(argv[2]), cost = atoi(argv[3]), tpw = atoi(argv[4]), repeat = atoi(argv[5]);
    Options o;
    {
        const std::string self(argv[0]);
        const std::string tail("_fp16");
        if (self.size() >= tail.size() && self.compare(self.size() - tail.size(), tail.size(), tail) == 0) o.dtype = "f16";
    }
    for (int i = 6; i < argc; ++i)
        if (!parse_option(argv[i], o)) { fprintf(stderr, "unknown or malformed option %s\n", argv[i]); return 2; }

    mps_csr g;
    {   // the reference's text file, or this library's binary sidecar of the same graph (recognised by its first bytes)
        char magic[8] = {0};
        if (FILE *f = fopen(argv[1], "rb")) { if (fread(magic, 1, 8, f) != 8) magic[0] = 0; fclose(f); }
        const bool sidecar = memcmp(magic, "MPSCSR01", 8) == 0;
        const int rc = sidecar ? mps_csr_load_bin(argv[1], &g, nullptr, nullptr) : mps_csr_load(argv[1], 0, &g);
        if (rc != MPS_OK) { fprintf(stderr, "error: %s\n", mps_last_error()); return 1; }
    }
    std::cout << "Total number of rows: " << g.n_rows << " and non-zeros: " << g.nnz << std::endl;
    if (dim < 1 || cost < 1) { fprintf(stderr, "error: dimension and cost must be >= 1\n"); return 2; }
    if (dim <= 32 && tpw > 32 / dim)
        fprintf(stderr, "note: threads_per_warp %d exceeds 32/dim = %d; using %d (the reference exits here)\n", tpw, 32 / dim, 32 / dim);
    const bool half = o.dtype == "f16";

    // values: none in the file; --values=gcn derives D^-1/2 (A) D^-1/2 from the row lengths
    std::vector<float> val;
    std::vector<__half> val_h;
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
        if (half) {
            val_h.resize(val.size());
            for (size_t k = 0; k < val.size(); ++k) val_h[k] = __float2half(val[k]);
        }
    }
    const void *val_ptr = val.empty() ? nullptr : (half ? (const void *)val_h.data() : (const void *)val.data());

    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess || visible < 1) { fprintf(stderr, "error: no CUDA device\n"); return 1; }
    if (o.gpus > visible) { fprintf(stderr, "error: --gpus=%d but only %d devices are visible\n", o.gpus, visible); return 1; }
    std::vector<int32_t> devices((size_t)o.gpus);
    for (int d = 0; d < o.gpus; ++d) devices[(size_t)d] = o.gpus == 1 ? o.device : d;

    // B = 1 everywhere, as the reference fills it (src/MergePathSpMM.cu:180-182)
    const size_t cells = (size_t)g.n_rows * dim, es = half ? 2 : 4;
    std::vector<unsigned char> hB(cells * es), hC(cells * es);
    if (half) { const __half one = __float2half(1.0f); for (size_t i = 0; i < cells; ++i) ((__half *)hB.data())[i] = one; }
    else for (size_t i = 0; i < cells; ++i) ((float *)hB.data())[i] = 1.0f;

    mps_multi *m = nullptr;
    auto t0 = std::chrono::steady_clock::now();
    MPS_OK_OR_DIE(mps_multi_create(o.gpus, devices.data(), g.n_rows, g.n_rows, dim, half ? MPS_F16 : MPS_F32, cost, tpw, g.row_ptr, g.col_idx,
                                   val_ptr, &m));
    const double setup_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    MPS_OK_OR_DIE(mps_multi_set_b(m, hB.data()));  // the first call also creates the communicator
    t0 = std::chrono::steady_clock::now();
    MPS_OK_OR_DIE(mps_multi_set_b(m, hB.data()));
    const double set_b_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    float ms = 0, ms_gather = 0;
    MPS_OK_OR_DIE(mps_multi_spmm(m, 3, 0, &ms, nullptr));  // warm-up
    if (repeat > 0) MPS_OK_OR_DIE(mps_multi_spmm(m, repeat, o.gather_c ? 1 : 0, &ms, &ms_gather));

    long long bad = 0;
    if (o.check) {  // with B == 1 every element of row i is the sum of the row's values
        MPS_OK_OR_DIE(mps_multi_get_c(m, hC.data(), o.gather_c ? o.gpus - 1 : -1));
        for (int i = 0; i < g.n_rows; ++i) {
            double want = 0;
            for (int k = g.row_ptr[i]; k < g.row_ptr[i + 1]; ++k)
                want += val.empty() ? 1.0 : (half ? (double)__half2float(val_h[(size_t)k]) : (double)val[(size_t)k]);
            const double tol = (half ? 1e-2 : 1e-5) * std::fabs(want) + 1e-6;
            for (int j = 0; j < dim; ++j) {
                const size_t at = (size_t)i * dim + j;
                const double got = half ? (double)half_to_float(((const uint16_t *)hC.data())[at]) : (double)((const float *)hC.data())[at];
                if (std::fabs(got - want) > tol) ++bad;
            }
        }
    }
    const double flops = 2.0 * g.nnz * dim;
    const double bytes = (double)mps_algorithmic_bytes(g.n_rows, g.nnz, dim, half ? MPS_F16 : MPS_F32, o.values == "gcn");
    printf("gpus: %d  dtype: %s  values: %s  dim: %d  cost: %d  repeat: %d\n", o.gpus, o.dtype.c_str(), o.values.c_str(), dim, cost, repeat);
    for (int d = 0; d < o.gpus; ++d) {
        int32_t dev, r0, r1, nz;
        mps_multi_slab(m, d, &dev, &r0, &r1, &nz, nullptr);
        printf("  device %d: rows [%d, %d)  nnz %d\n", dev, r0, r1, nz);
    }
    printf("upload + partition: %.3f ms (once)\n", setup_ms);
    printf("B to every device: %.3f ms (%.1f MB; %s)\n", set_b_ms, (double)(cells * es) / 1e6,
           o.gpus > 1 ? "each device uploads 1/gpus of the rows, NCCL all-gather completes them" : "one upload");
    if (repeat > 0)
        printf("time per SpMM: %.4f ms  %.1f GFLOP/s  %.1f GB/s algorithmic (max over devices)\n", ms, flops / ms / 1e6, bytes / ms / 1e6);
    if (o.gather_c) printf("all-gather of C over NCCL: %.4f ms\n", ms_gather);
    if (o.check) printf("check: %lld elements outside tolerance\n", bad);
    mps_multi_destroy(m);
    mps_csr_free(&g);
    return bad ? 3 : 0;
}
