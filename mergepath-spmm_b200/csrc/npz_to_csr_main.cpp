// npz_to_csr --graph <file.npz> --output <file.csr>
//
// Command-line twin of the reference's scripts/npz_to_csr.py (same two options, :8-11): reads the
// members src_li / dst_li of a GNNAdvisor-style .npz, builds the CSR structure scipy's tocsr() would
// (duplicates collapsed, columns sorted) and writes the two-line `.csr` text the SpMM programs read.
#include <cstdio>
#include <cstring>

#include "mps.h"

int main(int argc, char *argv[]) {
    const char *graph = nullptr, *output = nullptr;
    for (int i = 1; i + 1 < argc; i += 2) {
        if (!strcmp(argv[i], "--graph")) graph = argv[i + 1];
        else if (!strcmp(argv[i], "--output")) output = argv[i + 1];
    }
    if (!graph || !output) {
        fprintf(stderr, "usage: npz_to_csr --graph <file.npz> --output <file.csr>\n");
        return 2;
    }
    mps_csr csr;
    if (mps_npz_to_csr(graph, 0, &csr) != MPS_OK || mps_csr_save(output, csr.n_rows, csr.row_ptr, csr.col_idx) != MPS_OK) {
        fprintf(stderr, "error: %s\n", mps_last_error());
        return 1;
    }
    printf("%s: %d rows, %d non-zeros -> %s\n", graph, csr.n_rows, csr.nnz, output);
    mps_csr_free(&csr);
    return 0;
}
