// Chooses the kernel family for each call from the plan's diagonal pattern and the operands'
// alignment.
#include "cuvdia_internal.cuh"

namespace cuvdia {

int launch_prod(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                bool trans, float factAB, float factC, int mode, const ProdEpilogue* ep, cudaStream_t st) {
    int rc;
    // few diagonals or few columns: the streaming kernel if the band has at most 16 diagonals; wider bands are
    // better served by the run-walking kernel (TMA ring) than by the per-thread loads of the narrow kernel
    const bool runs = prod_runs_applicable(p, A, B, ldb);
    if (prod_narrow_applicable(p, A, B, ldb, ncols) && (prod_narrow_streams(p, trans) || !runs))
        rc = launch_prod_narrow(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    // (with fewer than 96 columns the tiled kernel's 128-column tile is mostly empty: the run-walking kernel is up to
    // 1.5 times faster at 64 columns and bands of 24-128 diagonals, and slower from 256 columns on)
    else if (!(runs && ncols < 96) && prod_band_applicable(p, A, B, ldb, ncols))
        rc = launch_prod_band(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    // steep bands (row factor 2, 4, 8) times many columns: the streaming banded kernel
    else if (prod_bandw_applicable(p, A, B, ldb, ncols))
        rc = launch_prod_bandw(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    else if (runs)
        rc = launch_prod_runs(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    else if (prod_windown_applicable(p, trans, A, B, ldb, ncols))
        rc = launch_prod_windown(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    else if (prod_window_applicable(p, trans, ncols))
        rc = launch_prod_window(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    else
        rc = launch_prod_generic(p, A, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, st);
    if (rc || !ep) return rc;
    // The element-wise tail runs as a second, bandwidth-bound pass over C.  Applying it inside the banded
    // kernel's epilogue was measured slower: with one block per SM the loads of the uniform numbers and
    // the exponentials at the end of every block are not overlapped with any other block's arithmetic.
    return launch_bias_sigmoid_sample(C, ldc, ep->bias, ep->U, ep->ldu, ep->S, ep->lds, trans ? p->w : p->h, ncols, st);
}

int launch_dd2dia(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                  float factAB, float factC, cudaStream_t st) {
    if (dd2dia_stream_applicable(p, Cv, A, lda, B, ldb, ncols))
        return launch_dd2dia_stream(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    // A narrow band times few batch columns is mostly padding in 128 x 128 tiles (two tiles per row block for 24
    // diagonals compute ten times what is stored): the run-aware kernel, which treats the band as runs of 8 diagonals
    // and is bound by memory, is up to 3.8 times faster there (131072 rows, 24 diagonals, 16 columns: 43 -> 12 us)
    // and loses from about 6000 diagonal-columns on.
    if (((long long)p->nd * ncols <= 6144 || (p->nd <= 32 && ncols <= 256)) && p->is_band &&
        dd2dia_runs_applicable(p, Cv, A, lda, B, ldb, ncols))
        return launch_dd2dia_runs(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    if (dd2dia_band_applicable(p, A, lda, B, ldb, ncols))
        return launch_dd2dia_band(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    // runs of consecutive diagonals (convolution patterns): every run a narrow band of its own
    if (dd2dia_runs_applicable(p, Cv, A, lda, B, ldb, ncols))
        return launch_dd2dia_runs(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    if (dd2dia_window_applicable(p, A, lda, B, ldb, ncols))
        return launch_dd2dia_window(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
    return launch_dd2dia_generic(p, Cv, A, lda, B, ldb, ncols, factAB, factC, st);
}

}  // namespace cuvdia
