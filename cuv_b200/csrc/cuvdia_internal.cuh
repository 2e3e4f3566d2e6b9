// Internal declarations shared by the translation units of libcuvdia.so.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "cuvdia.h"

namespace cuvdia {

// ---- error plumbing ---------------------------------------------------------------------------
void set_last_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define CUVDIA_REQUIRE(cond)                                                           \
    do {                                                                               \
        if (!(cond)) { ::cuvdia::set_last_error("%s", #cond); return CUVDIA_ERR_INVALID; } \
    } while (0)

#define CUVDIA_CUDA(call)                                                              \
    do {                                                                               \
        cudaError_t e__ = (call);                                                      \
        if (e__ != cudaSuccess) return ::cuvdia::cuda_fail(e__, #call);                \
    } while (0)

extern std::atomic<unsigned long long> g_launches;
inline void count_launch(unsigned n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
// Checks the launch that was just issued (configuration errors surface here, not at the next sync).
int check_launch(const char* kernel);

// ---- per-(device, stream) workspace for kernels that have no plan (reductions) -------------------
// Grows on demand with cudaMalloc; contents are undefined between calls.
int get_workspace(cudaStream_t stream, size_t bytes, void** ptr);

int sm_count();

// The TMA kernels need cuTensorMapEncodeTiled from the driver; false if it cannot be resolved (they are then not
// chosen and the kernels with plain loads run).
bool tma_available();

// Raises a kernel's dynamic shared-memory limit once per device (the attribute belongs to the device's
// context, so a process that uses several GPUs must set it on each).
template <class K>
inline int allow_dynamic_smem(K kernel, size_t bytes, bool (&done)[64]) {
    int dev = 0;
    CUVDIA_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { set_last_error("device index %d out of range", dev); return CUVDIA_ERR_UNSUPPORTED; }
    if (!done[dev]) {
        CUVDIA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        done[dev] = true;
    }
    return CUVDIA_OK;
}

}  // namespace cuvdia

// ---- plan ------------------------------------------------------------------------------------------
struct cuvdia_plan {
    int h, w, nd, stride, rf;
    int device;
    std::vector<int> offsets;   // storage (user) order
    int* d_offsets;             // device copy, storage order
    bool is_band;               // offsets[k] == offsets[0] + k
    int band_lo;                // offsets[0] when is_band
    int off_min, off_max;
    long long nnz;
    // scratch for densedense_to_dia's batch split (floats); allocated on first need
    float* scratch;
    size_t scratch_floats;
    // device word set non-zero by a kernel whose bounded wait on a TMA barrier gave up
    int* d_status;
    // the offset list cut, in storage order, into passes of up to 8 consecutive diagonal numbers:
    // (first slot, first offset, count, 0) per pass; on the device only when the pattern is made of runs
    bool is_runs;
    int npass;
    int* d_passes;
    // the diagonals in ascending order of their offsets: nd storage slots followed by nd offsets (device), and the
    // largest number of dense rows that 16 ([0]) and 32 ([1]) neighbours in that order span
    int* d_sorted;
    // the windowed densedense_to_dia's list of (row tile, group of neighbouring diagonals) pairs, three ints each
    // (device), their number and the diagonals they hold in total
    int* d_witems;
    int n_witems;
    long long witem_diagonals;
    // side stream (highest priority) and events of the step that overlaps its all-reduce; created on first use
    cudaStream_t side_stream;
    cudaEvent_t ev_first, ev_side;
};

namespace cuvdia {
// Which uniform numbers a pass draws: key (the seed's two halves), the draw within the step, the step, and the global
// index of the first batch column the call sees (see glue.cu).
struct DrawParams {
    unsigned k0, k1, which, step;
    long long col0;
};
inline DrawParams make_draw(const cuvdia_draw* d, unsigned which) {
    DrawParams r;
    r.k0 = (unsigned)(d->seed & 0xffffffffull); r.k1 = (unsigned)(d->seed >> 32);
    r.which = which; r.step = (unsigned)d->step; r.col0 = d->col0;
    return r;
}
// Optional element-wise tail of prod: C <- sigmoid(C + bias[row]); S <- C > U ? 1 : 0.
struct ProdEpilogue {
    const float* bias;       // may be null
    const float* U; int ldu; // null: no sampling
    float* S; int lds;
};
// kernels' host-side launchers (each returns a CUVDIA_* code)
int launch_prod(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                bool trans, float factAB, float factC, int mode, const ProdEpilogue* ep, cudaStream_t st);
int launch_dd2dia(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                  float factAB, float factC, cudaStream_t st);
int launch_prod_generic(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                        bool trans, float factAB, float factC, int mode, cudaStream_t st);
int launch_dd2dia_generic(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                          float factAB, float factC, cudaStream_t st);
int ensure_plan_scratch(cuvdia_plan* p, size_t floats, cudaStream_t st);
bool prod_band_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols);
int launch_prod_band(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                     bool trans, float factAB, float factC, int mode, cudaStream_t st);
bool prod_bandw_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols);
int launch_prod_bandw(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                      bool trans, float factAB, float factC, int mode, cudaStream_t st);
bool prod_narrow_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols);
// true if launch_prod_narrow would take its TMA streaming variant (at most 16 diagonals, many rows)
bool prod_narrow_streams(const cuvdia_plan* p, bool trans);
int launch_prod_narrow(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                       bool trans, float factAB, float factC, int mode, cudaStream_t st);
bool prod_runs_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb);
int launch_prod_runs(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                     bool trans, float factAB, float factC, int mode, cudaStream_t st);
// the staged-window kernel for row factor 1 with a lean inner loop (prod_windown.cu)
bool prod_windown_applicable(const cuvdia_plan* p, bool trans, const float* A, const float* B, int ldb, int ncols);
int launch_prod_windown(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                        bool trans, float factAB, float factC, int mode, cudaStream_t st);
bool prod_window_applicable(const cuvdia_plan* p, bool trans, int ncols);
int launch_prod_window(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                       bool trans, float factAB, float factC, int mode, cudaStream_t st);
bool dd2dia_stream_applicable(const cuvdia_plan* p, const float* Cv, const float* A, int lda, const float* B, int ldb,
                              int ncols);
int launch_dd2dia_stream(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float factAB, float factC, cudaStream_t st);
bool dd2dia_runs_applicable(const cuvdia_plan* p, const float* Cv, const float* A, int lda, const float* B, int ldb,
                            int ncols);
int launch_dd2dia_runs(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                       float factAB, float factC, cudaStream_t st);
bool dd2dia_window_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols);
int launch_dd2dia_window(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float factAB, float factC, cudaStream_t st);
bool dd2dia_band_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols);
int launch_dd2dia_band(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                       float factAB, float factC, cudaStream_t st);
// the (row tile, diagonal group) pairs of the windowed densedense_to_dia (see dd2dia_window.cu)
void window_items(int h, int w, int nd, int rf, const int* sorted_off, std::vector<int>* items);
// the banded densedense_to_dia cut in two launches by column tiles (see dd2dia_band.cu)
int dd2dia_band_cut(const cuvdia_plan* p, int ncols, int* first_diagonals, bool force);
int dd2dia_band_nsplit(const cuvdia_plan* p, int ncols);
int launch_dd2dia_band_range(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                             float factAB, float factC, int tile0, int tile1, cudaStream_t st);
int launch_reduce(float* dst, const float* src, long long n_contig, long long n_strided, bool over_strided,
                  int functor, float factNew, float factOld, cudaStream_t st);
int launch_reduce_typed(void* dst, int dst_type, const void* src, int src_type, long long n_contig, long long n_strided,
                        bool over_strided, int functor, float fnew, float fold, cudaStream_t st);
int launch_avg_diagonals(const cuvdia_plan* p, const float* A, float* dst, cudaStream_t st);
int launch_bias_sigmoid_sample(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                               int lds, int units, int ncols, cudaStream_t st);
// the same pass that also accumulates sum_dst[unit] = fold*sum_dst[unit] + fnew*sum over columns of the activation
// (sum_sample == 0) or of the 0/1 sample (sum_sample != 0); store_act == 0 leaves act unwritten
// draw != null: the uniform numbers are drawn in the kernel (u is not read)
int launch_bias_sigmoid_sample_sum(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                                   int lds, int units, int ncols, float* sum_dst, int sum_sample, float fnew, float fold,
                                   int store_act, cudaStream_t st, const DrawParams* draw = nullptr);
// dst[row, col] = the uniform number of (row, d.col0 + col) of draw d.which in step d.step
int launch_uniform(float* dst, int ld, int rows, int ncols, const DrawParams& d, cudaStream_t st);
// act[row, col] = act[row, col] > that number ? 1 : 0, in place
int launch_binarize(float* act, int ld, int rows, int ncols, const DrawParams& d, cudaStream_t st);
int launch_reduce_combine_add(float* dst, long long n_out, float fnew, float fold, int nsplit, const float* partial,
                              cudaStream_t st);
int launch_axpby(float* dst, const float* x, const float* y, float a, float b, long long n, cudaStream_t st);
// momentum-free when M is null: (a, b) = (alpha, beta); with momentum (a, b, c) = (lr, momentum weight, l2 decay)
int launch_learn_step(float* W, float* M, const float* dW, float a, float b, float c, long long n, cudaStream_t st);
int launch_binary(float* dst, const float* x, const float* y, int op, float p, float p2, long long n, cudaStream_t st);
int launch_fill(float* dst, float value, int sequence, long long n, cudaStream_t st);
int launch_selftest_wait(int* status, unsigned max_polls, cudaStream_t st);
}  // namespace cuvdia
