// cuSPARSE baseline, set up the way the reference's comparison programs do it
// (src/cusparse_spmm_row.cu:167-202, src/cusparse_spmm_col.cu:172-176): CSR with 32-bit indices and
// fp32 values, dense B and C row-major (leading dimension = dim) or column-major (leading dimension
// = rows), alpha = 1, beta = 0, CUSPARSE_SPMM_ALG_DEFAULT, external buffer from
// cusparseSpMM_bufferSize, no preprocess.  Those programs time an asynchronous call with
// std::chrono and no synchronisation (:193-208); here CUDA events bracket `repeat` calls.
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY (a reported baseline, never shipped).
#include <cuda_runtime.h>
#include <cusparse.h>

#define CUSH_API extern "C" __attribute__((visibility("default")))

// col_major != 0: B is n_cols x dim and C is n_rows x dim stored column-major.  alg: 0 =
// CUSPARSE_SPMM_ALG_DEFAULT as the reference uses it; 1, 2, 3 = CUSPARSE_SPMM_CSR_ALG1/2/3 with
// cusparseSpMM_preprocess (a fairer library baseline than the reference's set-up).  Returns 0 and the
// mean milliseconds per SpMM in *ms, or a negative step number on failure.
CUSH_API int cush_spmm(int n_rows, int n_cols, int nnz, int dim, const int *d_rp, const int *d_col, const float *d_val,
                       const float *d_B, float *d_C, int col_major, int alg_id, int repeat, float *ms) {
    const cusparseSpMMAlg_t alg = alg_id == 1 ? CUSPARSE_SPMM_CSR_ALG1 : alg_id == 2 ? CUSPARSE_SPMM_CSR_ALG2
                                  : alg_id == 3 ? CUSPARSE_SPMM_CSR_ALG3 : CUSPARSE_SPMM_ALG_DEFAULT;
    cusparseHandle_t h = nullptr;
    cusparseSpMatDescr_t A = nullptr;
    cusparseDnMatDescr_t B = nullptr, C = nullptr;
    void *buf = nullptr;
    size_t buf_bytes = 0;
    const float alpha = 1.0f, beta = 0.0f;
    int rc = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cusparseCreate(&h) != CUSPARSE_STATUS_SUCCESS) return -1;
    if (cusparseCreateCsr(&A, n_rows, n_cols, nnz, (void *)d_rp, (void *)d_col, (void *)d_val, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I,
                          CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F) != CUSPARSE_STATUS_SUCCESS) rc = -2;
    const cusparseOrder_t order = col_major ? CUSPARSE_ORDER_COL : CUSPARSE_ORDER_ROW;
    if (!rc && cusparseCreateDnMat(&B, n_cols, dim, col_major ? n_cols : dim, (void *)d_B, CUDA_R_32F, order) != CUSPARSE_STATUS_SUCCESS) rc = -3;
    if (!rc && cusparseCreateDnMat(&C, n_rows, dim, col_major ? n_rows : dim, (void *)d_C, CUDA_R_32F, order) != CUSPARSE_STATUS_SUCCESS) rc = -4;
    if (!rc && cusparseSpMM_bufferSize(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, C, CUDA_R_32F,
                                       alg, &buf_bytes) != CUSPARSE_STATUS_SUCCESS) rc = -5;
    if (!rc && cudaMalloc(&buf, buf_bytes ? buf_bytes : 16) != cudaSuccess) rc = -6;
    if (!rc && alg_id != 0 &&
        cusparseSpMM_preprocess(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, C, CUDA_R_32F, alg,
                                buf) != CUSPARSE_STATUS_SUCCESS) rc = -10;
    if (!rc) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        for (int i = 0; i < 2 && !rc; ++i)  // warm-up
            if (cusparseSpMM(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, C, CUDA_R_32F,
                             alg, buf) != CUSPARSE_STATUS_SUCCESS) rc = -7;
        cudaDeviceSynchronize();
        cudaEventRecord(e0);
        for (int i = 0; i < repeat && !rc; ++i)
            if (cusparseSpMM(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, B, &beta, C, CUDA_R_32F,
                             alg, buf) != CUSPARSE_STATUS_SUCCESS) rc = -8;
        cudaEventRecord(e1);
        if (cudaDeviceSynchronize() != cudaSuccess) rc = -9;
        float t = 0.0f;
        if (!rc) { cudaEventElapsedTime(&t, e0, e1); *ms = t / (repeat > 0 ? repeat : 1); }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    cudaFree(buf);
    if (C) cusparseDestroyDnMat(C);
    if (B) cusparseDestroyDnMat(B);
    if (A) cusparseDestroySpMat(A);
    cusparseDestroy(h);
    return rc;
}
