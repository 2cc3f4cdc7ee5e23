/*
 * TEST INFRASTRUCTURE - CPU oracle for the sparse x dense product of the broadcast-SpMM path.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may link or call
 * this file; the product never does.
 *
 * What it restates.  The reference multiplies one coalesced COO block by a dense row-major fp32
 * matrix and accumulates in place, either through cuSPARSE
 * (light_dist_gnn/spmm_cpp/spmm.cpp:17-33, C = alpha*A*B + beta*C, int32 indices, row-major
 * operands) or through torch's sparse addmm_ on the CPU (light_dist_gnn/models/gcn.py:13).  The
 * arithmetic of both lives in third-party libraries that are not part of the reference tree
 * (cuSPARSE 11/12; PyTorch, no version pinned by the reference, 2.11.0 in this image).  The
 * published semantics restated here: for a coalesced COO (entries sorted by row, then column, no
 * duplicates) every output row is  beta*C[i,:] + alpha * sum_j A[i,j]*B[j,:], the sum taken in
 * ascending column order in fp32 with a separate multiply and add per term.
 *
 * Parity status: pinned by outputs of the reference's own CPU path (C.addmm_(A, B) and the whole
 * gloo stage loop) generated in the build container and stored under tests/golden/.
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp -ffp-contract=off; outputs in oracle/_build/).
 */
#include <stdint.h>
#include <stddef.h>

/* rowptr[i] = number of entries with row < i; rows must be sorted ascending. */
void oracle_coo_to_rowptr(const int32_t *row, int64_t nnz, int32_t m, int64_t *rowptr)
{
    int64_t e = 0;
    for (int32_t i = 0; i <= m; ++i) {
        while (e < nnz && row[e] < i) ++e;
        rowptr[i] = e;
    }
}

/* C = alpha*A*B + beta*C for a CSR block (rowptr int64 [m+1], col int32, val fp32), B [k x F] with
 * leading dimension ldb, C [m x F] with leading dimension ldc.  beta == 0 overwrites C without
 * reading it (so NaNs in an uninitialised C do not propagate, as in cuSPARSE).  Rows are
 * independent, so the OpenMP split does not change any sum order. */
void oracle_spmm_csr(const int64_t *rowptr, const int32_t *col, const float *val, int32_t m,
                     const float *B, int64_t ldb, float *C, int64_t ldc, int32_t F,
                     float alpha, float beta, int threads)
{
    (void)threads;
#pragma omp parallel for schedule(dynamic, 64) num_threads(threads > 0 ? threads : 1)
    for (int32_t i = 0; i < m; ++i) {
        float *c = C + (size_t)i * ldc;
        for (int32_t f0 = 0; f0 < F; f0 += 64) {          /* column strip keeps acc[] in registers/L1 */
            int32_t w = F - f0 < 64 ? F - f0 : 64;
            float acc[64];
            for (int32_t f = 0; f < w; ++f) acc[f] = 0.0f;
            for (int64_t e = rowptr[i]; e < rowptr[i + 1]; ++e) {
                const float a = val[e];
                const float *b = B + (size_t)col[e] * ldb + f0;
                for (int32_t f = 0; f < w; ++f) acc[f] = acc[f] + a * b[f];
            }
            if (beta == 0.0f)
                for (int32_t f = 0; f < w; ++f) c[f0 + f] = alpha * acc[f];
            else
                for (int32_t f = 0; f < w; ++f) c[f0 + f] = alpha * acc[f] + beta * c[f0 + f];
        }
    }
}

/* The 9-argument COO form of spmm.cpp:17 (row/col/val + dims + B + C + alpha + beta), F = width of B and C. */
void oracle_spmm_coo(const int32_t *row, const int32_t *col, const float *val, int64_t nnz,
                     int32_t m, int32_t k, const float *B, float *C, int32_t F,
                     float alpha, float beta, int64_t *rowptr_scratch, int threads)
{
    (void)k;
    oracle_coo_to_rowptr(row, nnz, m, rowptr_scratch);
    oracle_spmm_csr(rowptr_scratch, col, val, m, B, F, C, F, F, alpha, beta, threads);
}
