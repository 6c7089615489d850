// Shared by the translation units of libmps_b200.so; not part of the public ABI.
#pragma once
#include <stdint.h>

#include "mps.h"

namespace mps {
// Records a printf-style message for mps_last_error() on this thread and returns `code`.
int fail(int code, const char *fmt, ...);

// Host-side scans of a caller's CSR (host_check.cpp), each on up to `threads` host threads (0 = all):
// index of the first row whose row_ptr decreases / of the first column index outside [0, n_cols), or -1.
long long first_decreasing_row(const int32_t *row_ptr, long long n_rows, int threads);
long long first_bad_column(const int32_t *col_idx, long long nnz, int32_t n_cols, int threads);
int32_t max_column(const int32_t *col_idx, long long nnz, int threads);
// row_ptr[0] == 0, row_ptr non-decreasing, every column index inside [0, n_cols) (col_idx may be NULL): MPS_OK or
// MPS_ERR_ARG with the offending position in the message.
int check_csr_host(const char *who, int32_t n_rows, int32_t n_cols, const int32_t *row_ptr, const int32_t *col_idx, int threads);
}  // namespace mps
