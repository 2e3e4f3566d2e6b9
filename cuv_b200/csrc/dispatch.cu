// Chooses the kernel family for each call from the plan's diagonal pattern and the operands'
// alignment.
#include "cuvdia_internal.cuh"

namespace cuvdia {

int launch_prod(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                bool trans, float factAB, float factC, int mode, cudaStream_t st) {
    if (prod_band_applicable(p, A, B, ldb, ncols))
        return launch_prod_band(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    if (prod_window_applicable(p, trans, ncols))
        return launch_prod_window(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    return launch_prod_generic(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
}

int launch_dd2dia(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                  float factAB, float factC, cudaStream_t st) {
    if (dd2dia_band_applicable(p, A, lda, B, ldb, ncols))
        return launch_dd2dia_band(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    return launch_dd2dia_generic(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
}

}  // namespace cuvdia
