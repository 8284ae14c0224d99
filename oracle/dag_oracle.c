/*
 * oracle/dag_oracle.c — CPU oracle for the DAG custom ops (plain C, OpenMP over
 * sentences / rows).
 *
 * TEST INFRASTRUCTURE ONLY.  It is the checker, never the product: only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Parity pin: this restatement is checked against golden vectors produced by
 * importing the reference's own torch-native functions (torch_dag_loss,
 * torch_dag_best_alignment, torch_dag_logsoftmax_gather_inplace of
 * fs_plugins/custom_ops/dag_loss.py:259-359) — see tests/golden/make_golden.py — and, for
 * the functions of graph_oracle_impl.inc (forced alignment, extract_links tail, decode-side
 * dynamic programmes), by running the reference's own method bodies — see
 * tests/golden/make_golden_graph.py.
 * The reference has no golden vectors of its own, and the reduction order of its
 * CUDA kernels is not pinned by any reference test, so bit-level parity of the
 * floating-point results is unpinned; they are pinned to tolerances.  The
 * alignment tie-break is restated literally from the CUDA kernel.
 *
 * Build: see oracle/Makefile  (gcc -O2 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define REAL double
#define SFX _f64
#define EXP exp
#define LOG log
#include "dag_oracle_impl.inc"
#include "graph_oracle_impl.inc"
#undef REAL
#undef SFX
#undef EXP
#undef LOG

#define REAL float
#define SFX _f32
#define EXP expf
#define LOG logf
#include "dag_oracle_impl.inc"
#include "graph_oracle_impl.inc"
#undef REAL
#undef SFX
#undef EXP
#undef LOG

/* band <-> square link layouts: fs_plugins/models/glat_decomposed_with_link.py:319-349
 * and fs_plugins/custom_ops/dag_loss.py:373-382.
 *   band[b,i,d] = square[b,i,i+d+1]   (-inf past the end) */
void oracle_band_to_square_f64(const double *band, int B, int L, int K, double *sq) {
    for (size_t x = 0; x < (size_t)B * L * L; x++) sq[x] = -INFINITY;
    for (int b = 0; b < B; b++)
        for (int i = 0; i < L; i++)
            for (int d = 0; d < K; d++) {
                int j = i + d + 1;
                if (j < L) sq[((size_t)b * L + i) * L + j] = band[((size_t)b * L + i) * K + d];
            }
}

void oracle_square_to_band_f64(const double *sq, int B, int L, int K, double *band) {
    for (int b = 0; b < B; b++)
        for (int i = 0; i < L; i++)
            for (int d = 0; d < K; d++) {
                int j = i + d + 1;
                band[((size_t)b * L + i) * K + d] =
                    j < L ? sq[((size_t)b * L + i) * L + j] : -INFINITY;
            }
}

int oracle_abi_version(void) { return 2; }

/* Number of OpenMP threads the parallel loops will use; n > 0 sets it first (launchers such as
 * torchrun export OMP_NUM_THREADS=1, which would silently make a "32 thread" baseline single-threaded). */
int oracle_set_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
}
