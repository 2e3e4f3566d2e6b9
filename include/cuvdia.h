/*
 * cuvdia.h - C ABI of the B200 (sm_100a) implementation of CUV's DIA sparse hot path.
 *
 * Every entry point below replaces one device_memory_space routine of CUV; the comment on each
 * names the reference interface (file:line within the CUV source tree) whose FFI it is.  CUV's
 * C++ templates (include/cuv/...) forward their dev_memory_space specialisations to these calls.
 *
 * Conventions
 *  - All matrix pointers are DEVICE pointers to fp32, column-major, with a leading dimension in
 *    elements.  `offsets_host` is a HOST pointer.  `stream` is a cudaStream_t passed as void*;
 *    NULL means the legacy default stream.  Calls are stream-ordered and do not synchronise
 *    (CUV's blocking behaviour is restored by the C++ wrappers, which synchronise afterwards).
 *  - Every function returns 0 on success or a CUVDIA_ERR_* code; cuvdia_error_string() names the
 *    code and cuvdia_last_error_message() gives the failed precondition of the calling thread's
 *    last failing call (the text CUV's cuvAssert would have thrown).  Preconditions are checked
 *    before anything is launched.
 *  - There is no CPU fallback: without a CUDA device every compute call fails with
 *    CUVDIA_ERR_CUDA.
 *  - Concurrency: a plan carries scratch memory (the batch split of densedense_to_dia) and the library keeps
 *    one workspace per (device, stream) for the split reductions; both grow on demand and are reused by the
 *    next call.  Use a plan from one stream and one host thread at a time, and a stream from one host thread
 *    at a time: two calls that share a plan or a stream's workspace and overlap on the GPU would overwrite each
 *    other's partial results.  Different plans on different streams are independent.
 *  - Waits inside the kernels (on asynchronous copies) are bounded.  A kernel that runs out of polls leaves its
 *    output incomplete and a non-zero code in the plan's health word; the calls below are stream-ordered and do
 *    not read that word, so callers of this C ABI poll cuvdia_plan_status() themselves (the C++ wrappers in
 *    include/cuv and cuv_b200's check_status=True do so after their synchronisation and throw, as CUV's
 *    blocking operations throw on failure, tools/cuv_general.cu:51-61).
 */
#ifndef CUVDIA_H
#define CUVDIA_H

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CUVDIA_API __attribute__((visibility("default")))
#else
#define CUVDIA_API
#endif

#define CUVDIA_OK               0
#define CUVDIA_ERR_INVALID      1   /* a precondition (CUV: cuvAssert) failed                      */
#define CUVDIA_ERR_CUDA         2   /* a CUDA runtime call failed (CUV: cuvSafeCall/checkCudaError) */
#define CUVDIA_ERR_UNSUPPORTED  3   /* valid in CUV's interface but not implemented here            */
#define CUVDIA_ERR_NOMEM        4   /* device or host allocation failed                             */

/* Arithmetic of prod.  EXACT evaluates every output in the order of CUV's host code
 * (matrix_ops/spmv.cu:153-198): separate multiply and add, diagonals in storage order, and is
 * bit-identical to it.  FAST fuses multiply and add (one rounding per term, same order). */
#define CUVDIA_MODE_EXACT 0
#define CUVDIA_MODE_FAST  1

/* Reduce functors: the values of enum cuv::reduce_functor, matrix_ops/matrix_ops.hpp:185-196. */
#define CUVDIA_RF_ADD          0
#define CUVDIA_RF_MEAN         1
#define CUVDIA_RF_ADD_SQUARED  2
#define CUVDIA_RF_MAX          3
#define CUVDIA_RF_ARGMAX       4
#define CUVDIA_RF_ARGMIN       5
#define CUVDIA_RF_MIN          6
#define CUVDIA_RF_MULT         7
#define CUVDIA_RF_LOGADDEXP    8
#define CUVDIA_RF_ADDEXP       9

CUVDIA_API const char* cuvdia_error_string(int code);
CUVDIA_API const char* cuvdia_last_error_message(void);

/* Number of kernels this library has launched in this process (all threads), for harnesses that
 * must prove the CUDA path ran. */
CUVDIA_API unsigned long long cuvdia_launch_count(void);

/* Frees the per-stream workspaces the library has allocated on the current device (the partial results of split
 * reductions and of the element-wise pass with batch sums); blocks until the device is idle first.  They are
 * re-created on demand.  No counterpart in CUV, whose allocations all belong to its tensors. */
CUVDIA_API int cuvdia_release_workspaces(void);

/* ---------------------------------------------------------------------------------------------
 * Plan: the structure of one DIA matrix (shape, diagonals, row factor) with the device-side
 * metadata and scratch the kernels need.  It replaces the internals of
 * cuv::dev_block_descriptor (matrix_ops/densedense_to_sparse.hpp:72-105, ctor
 * densedense_to_sparse.cu:123-171) and the per-call offset handling of spmv_dia_device
 * (matrix_ops/spmv.cu:89-101); like the block descriptor it can be reused for every matrix with
 * the same layout.  It never owns or reads matrix values.
 *
 * h, w        matrix height and width             (basics/matrix.hpp:49-106)
 * num_dia     number of stored diagonals          (basics/dia_matrix.hpp:76,146)
 * stride      floats per stored diagonal, >= h    (basics/dia_matrix.hpp:77,129-133; cells are
 *             indexed by the ROW of the matrix: value(i,j) = vals[slot*stride + i], :228-243)
 * row_fact    "steepness": diagonal k holds the cells (i, i/row_fact + k)   (:81,230)
 * offsets_host  num_dia diagonal numbers in the caller's order; the order is the storage order
 *             and is never changed (basics/dia_matrix.hpp:156-185).  A diagonal number may occur more
 *             than once, as in CUV (its speed fixture does that, src/tests/spmv_speed.cpp:96-104): prod
 *             sums every stored diagonal, densedense_to_dia fills every one of them, and element access
 *             (dia_matrix.hpp:181-185,236-243) sees the last.
 * The plan is bound to the CUDA device that is current when it is created.
 * ------------------------------------------------------------------------------------------- */
typedef struct cuvdia_plan cuvdia_plan;

CUVDIA_API int cuvdia_plan_create(cuvdia_plan** plan, int h, int w, int num_dia, int stride, int row_fact,
                       const int* offsets_host);
CUVDIA_API int cuvdia_plan_destroy(cuvdia_plan* plan);

/* Structure queries.  is_band: 1 when offsets are consecutive ascending integers in storage
 * order (the banded kernels apply).  nnz: number of matrix cells the stored diagonals cover
 * (sum over diagonals of N as in matrix_ops/spmv.cu:185-189). */
CUVDIA_API int cuvdia_plan_info(const cuvdia_plan* plan, int* is_band, long long* nnz);

/* Device-side health word of the plan, copied to *status (blocking: waits for the device).  0 = no
 * kernel of this plan ever gave up a bounded wait on an asynchronous copy; non-zero = one did and
 * its output is incomplete.  Waits inside the kernels are bounded so that a fault in the copy
 * engine cannot hang the GPU. */
CUVDIA_API int cuvdia_plan_status(const cuvdia_plan* plan, int* status);

/* Sets the plan's health word back to 0 (stream-ordered).  No counterpart in CUV. */
CUVDIA_API int cuvdia_plan_status_clear(cuvdia_plan* plan, void* stream);

/* Self-test of the bounded waits, no counterpart in CUV: launches one warp that waits, like the kernels of
 * this library do, for a copy-completion barrier - one that nothing will ever complete - gives up after
 * max_polls polls, writes the code 9 into the plan's health word and returns.  Nothing hangs and nothing
 * faults; afterwards cuvdia_plan_status reports 9 and the device is as usable as before. */
CUVDIA_API int cuvdia_selftest_bounded_wait(cuvdia_plan* plan, unsigned max_polls, void* stream);

/* Device pointer to the plan's copy of the offsets (int32, storage order), e.g. to initialise a
 * dia_matrix<float,dev_memory_space>::get_offsets() tensor. */
CUVDIA_API const int* cuvdia_plan_offsets_device(const cuvdia_plan* plan);

/* ---------------------------------------------------------------------------------------------
 * C = factC*C + factAB*op(A)*B with A in DIA format.
 * Replaces cuv::prod(tensor&, const dia_matrix<float,dev_memory_space>&, const tensor&, char,
 * char, const float&, const float&)  (matrix_ops/matrix_ops.hpp:118-119; device specialisation
 * matrix_ops/spmv.cu:221-247 and the generated dispatch it calls) and cuv::spmv
 * (matrix_ops/matrix_ops.hpp:277-278, spmv.cu:248-253), for any row_fact >= 1.
 *
 * transA 'n': B is w x ncols, C is h x ncols.   transA 't': B is h x ncols, C is w x ncols.
 * factC == 0 means C is overwritten and never read (spmv.cu:153-154).  Cells of A_vals outside
 * the range each diagonal covers are never read.  B and C must not overlap.
 * Errors (CUVDIA_ERR_INVALID), mirroring spmv.cu:211-214,229-240: transA not 'n'/'t', transB
 * not 'n', null pointers, ldb/ldc smaller than the row counts, ncols < 0.
 * ------------------------------------------------------------------------------------------- */
CUVDIA_API int cuvdia_prod_f32(const cuvdia_plan* plan, const float* A_vals,
                    const float* B, int ldb, float* C, int ldc, int ncols,
                    char transA, char transB, float factAB, float factC, int mode, void* stream);

/* ---------------------------------------------------------------------------------------------
 * C_dia = factC*C_dia + factAB*(A*B^T restricted to the stored diagonals).
 * Replaces cuv::densedense_to_dia(dia_matrix<float,dev_memory_space>&, const
 * dev_block_descriptor<float>&, const tensor&, const tensor&, const float&, const float&)
 * (matrix_ops/densedense_to_sparse.hpp:123-130; launcher densedense_to_sparse.cu:253-296, kernel
 * :51-120).  A is h x ncols, B is w x ncols.  factC == 0: C_dia cells are overwritten, not read;
 * cells outside each diagonal's range are neither read nor written (:104-119).  The sum over the
 * batch is evaluated in a fixed order, so repeated calls give identical bits.
 * Requires h % row_fact == 0 (the reference's host loop overruns otherwise, :244-249).
 * May allocate plan-owned scratch on first use (not during stream capture).
 * ------------------------------------------------------------------------------------------- */
CUVDIA_API int cuvdia_dd2dia_f32(cuvdia_plan* plan, float* C_vals, const float* A, int lda,
                      const float* B, int ldb, int ncols, float factAB, float factC, void* stream);

/* dst[k] = mean of stored diagonal k over the cells that lie inside the matrix (num_dia floats, device memory).
 * Replaces cuv::avg_diagonals(tensor&, const dia_matrix&) (matrix_ops/diagonals.hpp:12) with the definition of its
 * host code (matrix_ops/diagonals.cu:23-48; row_fact must be 1, :28).  CUV's device version (:13-22) averages the
 * whole stored array of each diagonal, padding included; the host definition is followed.  A diagonal with no cell
 * inside the matrix gives NaN.  The sum is taken in a fixed tree order (batch-sum tolerance). */
CUVDIA_API int cuvdia_avg_diagonals_f32(const cuvdia_plan* plan, const float* A_vals, float* dst, void* stream);

/* ---------------------------------------------------------------------------------------------
 * dst = factOld*dst + factNew*functor(src) along one axis of a matrix.
 * Replaces cuv::reduce_to_col / cuv::reduce_to_row (matrix_ops/matrix_ops.hpp:211-212,227-228;
 * layout dispatch matrix_ops_reduce.cu:348-379, device launchers :155-215, kernels :39-147).
 * src is n_strided lines of n_contig contiguous floats (a column-major n_contig x n_strided
 * matrix, or a row-major n_strided x n_contig one).
 *   over_strided != 0: reduce across lines; dst has n_contig entries
 *       (reduce_to_col of a column-major matrix, reduce_to_row of a row-major one);
 *   over_strided == 0: reduce along each line; dst has n_strided entries.
 * factOld == 0: dst is not read (:95-99,139-144).  ARGMAX/ARGMIN store the index as float and
 * ignore the factors; MEAN requires factNew == 1 and factOld == 0 (:308-313).
 * Uses a library-owned per-stream workspace that may be allocated on first use.
 * ------------------------------------------------------------------------------------------- */
CUVDIA_API int cuvdia_reduce_f32(float* dst, const float* src, long long n_contig, long long n_strided,
                      int over_strided, int functor, float factNew, float factOld, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The reduction between the other element types CUV instantiates (matrix_ops/matrix_ops_reduce.cu:395-413):
 * (source, destination) = (int, float), (unsigned, float), (unsigned char, float), (float, int),
 * (float, unsigned), (float, unsigned char), (unsigned char, unsigned char), (unsigned char, unsigned);
 * (float, float) forwards to cuvdia_reduce_f32; any other pair returns CUVDIA_ERR_UNSUPPORTED, as CUV has no
 * instantiation for it.  Semantics are those of CUV's code, which keeps the running value in the SOURCE type
 * and folds in the DESTINATION type (matrix_ops_reduce.cu:217-292, reduce_switch :304-343):
 *   ADD/MEAN r = (S)((D)r + (D)x);  ADD_SQUARED r = (S)((D)r + (D)(x*x));  MAX/MIN/ARGMAX/ARGMIN compare in S;
 *   dst = factOld*dst + factNew*r with both factors converted to S first (unsigned char: 0.5 becomes 0) and the
 *   expression evaluated by C++'s usual arithmetic conversions before it is stored as D; ARG* store the index;
 *   MEAN divides by the line length in D.
 * Integer running values wrap to the width of S (8 or 32 bits), so the result does not depend on the summation
 * order and is bit-identical to CUV's sequential host loop wherever C++ defines that loop (no float -> integer
 * conversion out of range, no signed overflow, sums routed through float below 2^24).  MULT, LOGADDEXP and
 * ADDEXP are float -> float only (CUVDIA_ERR_UNSUPPORTED otherwise).  Layout arguments as cuvdia_reduce_f32.
 * ------------------------------------------------------------------------------------------- */
#define CUVDIA_T_F32 0
#define CUVDIA_T_I32 1
#define CUVDIA_T_U32 2
#define CUVDIA_T_U8  3
CUVDIA_API int cuvdia_reduce(void* dst, int dst_type, const void* src, int src_type, long long n_contig,
                             long long n_strided, int over_strided, int functor, float factNew, float factOld,
                             void* stream);

/* ---------------------------------------------------------------------------------------------
 * The same reduction as cuvdia_reduce_f32 for callers that must not allocate device memory.
 * No counterpart in CUV; it exists because cuvdia_reduce_f32 may call cudaMalloc for its per-stream
 * workspace, and some callers cannot accept that: code that runs inside a fixed device-memory
 * budget given out by a host application, services that forbid allocator calls once they are up
 * (an allocation can stall every stream of the device), and callers with no chance to release what
 * a library allocated for them.  This entry point never calls cudaMalloc, cudaFree or any other
 * allocating routine.  The partial results of a split reduction live in a 4 MiB array that is part
 * of the library image (every device that loads the library holds it until the process exits).
 *  - Shapes whose split needs more than 4 MiB (8 bytes x partial results x outputs) are refused
 *    with CUVDIA_ERR_UNSUPPORTED and a message that states the need; use cuvdia_reduce_f32 then.
 *  - The first call on each device looks up the array's device address; make that first call
 *    outside any stream capture, with the device current.
 *  - All calls share the one array, which keeps the previous call's contents (nothing in it needs
 *    clearing: each call writes every slot it later reads).  Two calls that overlap on the GPU -
 *    different streams or different host threads - race on it; run them in one stream or
 *    serialise them.
 *  - It always takes the general split kernels; for very short lines, where cuvdia_reduce_f32 has
 *    sub-warp and grouped variants, it is slower than that entry point (same results).
 * Arguments, semantics and results are those of cuvdia_reduce_f32.
 * ------------------------------------------------------------------------------------------- */
CUVDIA_API int cuvdia_reduce_noalloc_f32(float* dst, const float* src, long long n_contig, long long n_strided,
                                         int over_strided, int functor, float factNew, float factOld,
                                         void* stream);

/* ---------------------------------------------------------------------------------------------
 * Element-wise glue of the RBM step on a column-major [units x ncols] activation matrix:
 *   act <- sigmoid(act + bias[unit])      (bias may be NULL)
 *   sample <- act > u ? 1 : 0             (sample and u may both be NULL)
 * Replaces the sequence matrix_plus_col (matrix_ops/matrix_ops.hpp:306-307), apply_scalar_functor
 * SF_SIGM (tensor_ops/functors.hpp:122) and rnd_binarize's compare (random/random.cu:86-91) that
 * examples/rbm/base.py:52-54,93-106 issues after each prod.
 * ------------------------------------------------------------------------------------------- */
CUVDIA_API int cuvdia_bias_sigmoid_sample_f32(float* act, int ld, const float* bias, const float* u, int ldu,
                                   float* sample, int lds, int units, int ncols, void* stream);

/* The same element-wise pass that also accumulates the per-unit sum over the batch columns it streams:
 *   sum_dst[unit] = factOld*sum_dst[unit] + factNew * sum_col x[unit, col]
 * with x = act after the logistic (sum_of_sample == 0) or x = sample (sum_of_sample != 0; sample required).
 * It replaces the reduce_to_col(dst, x, RF_ADD, factNew, factOld) that the RBM trainer issues afterwards for
 * its bias gradients (examples/rbm/base.py:76-83; reduce_to_col: matrix_ops/matrix_ops.hpp:211-212) - the matrix
 * is not read a second time.  factOld == 0: sum_dst is not read.  store_act == 0: act is not written back (for
 * callers that only use the sample and its sum; sample required).  The batch is summed in a fixed order
 * (reproducible run to run), not the host loop's sequential order: batch-sum tolerance as for cuvdia_reduce_f32.
 * act, sample are bit-identical to cuvdia_bias_sigmoid_sample_f32.  Uses the per-stream workspace. */
CUVDIA_API int cuvdia_bias_sigmoid_sample_sum_f32(float* act, int ld, const float* bias, const float* u, int ldu,
                                                  float* sample, int lds, int units, int ncols, float* sum_dst,
                                                  int sum_of_sample, float factNew, float factOld, int store_act,
                                                  void* stream);

/* prod followed by the element-wise tail of an RBM/MLP layer in one call:
 *   C <- sigmoid(factC*C + factAB*op(A)*B + bias[row]);   sample <- C > u ? 1 : 0   (u, sample may be NULL)
 * i.e. cuvdia_prod_f32 + cuvdia_bias_sigmoid_sample_f32, which is what upPass/downPass of
 * examples/rbm/base.py:48-54,93-106 issue back to back (prod, matrix_plus_col, SF_SIGM, rnd_binarize).
 * One entry point, two stream-ordered kernels (the product, then a bandwidth-bound pass over C);
 * results are identical to the two separate calls. */
CUVDIA_API int cuvdia_prod_bias_sigmoid_sample_f32(const cuvdia_plan* plan, const float* A_vals, const float* B,
                                                   int ldb, float* C, int ldc, int ncols, char transA, float factAB,
                                                   float factC, int mode, const float* bias, const float* u, int ldu,
                                                   float* sample, int lds, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One contrastive-divergence (CD-1) step of a sparse RBM whose weight matrix W (hidden x visible,
 * row_fact 1) is the plan's DIA matrix, queued on one stream.  No single CUV routine corresponds to
 * it: it issues, in the trainer's order (examples/rbm/base.py:223-258 with one Gibbs step; upPass /
 * downPass :48-54, gradient accumulation :76-83), the DIA forms of the calls made there:
 *   gb  =  1/B sum_b V0                                               (reduce_to_col)
 *   H0p = sigm(W V0 + c_hid),    H0 = H0p > U_h,   gc  =  1/B sum_b H0p   (prod 'n', one element-wise pass)
 *   V1p = sigm(W^T H0 + b_vis),  V1 = V1p > U_v,   gb -=  1/B sum_b V1    (prod 't', one element-wise pass)
 *   H1p = sigm(W V1 + c_hid),                      gc -=  1/B sum_b H1p   (prod 'n', one element-wise pass)
 *   G   =  1/B (H0p V0^T)|dia;   G += -1/B (H1p V1^T)|dia                 (densedense_to_dia x2)
 * All matrices are column-major with leading dimension = their row count (hidden: h, visible: w) and
 * ncols batch columns.  B = batch_global >= ncols: a rank that holds only its share of the batch
 * columns gets partial sums in G_vals, gc, gb, which cuvdia_allreduce_grad completes.  The uniform
 * numbers are inputs, so the step is deterministic.  keep_v1p == 0: V1p is left holding the
 * pre-activations (nothing after the sampling reads the probabilities).  Results are those of the
 * separate entry points called in this order.  May allocate scratch on first use (not during capture).
 * ------------------------------------------------------------------------------------------- */
typedef struct cuvdia_rbm_cd1_buffers {
    const float* V0;            /* visible data, w x ncols, values 0/1                     */
    const float* U_h;           /* uniform numbers for the hidden sample, h x ncols        */
    const float* U_v;           /* uniform numbers for the visible sample, w x ncols       */
    const float* b_vis;         /* visible bias, w floats, or NULL for zero                */
    const float* c_hid;         /* hidden bias, h floats, or NULL for zero                 */
    float* H0p; float* H0;      /* h x ncols: hidden probabilities and sample (outputs)    */
    float* V1p; float* V1;      /* w x ncols: reconstruction probabilities and sample      */
    float* H1p;                 /* h x ncols: hidden probabilities of the reconstruction   */
    float* G_vals;              /* num_dia*stride: weight gradient on W's diagonals        */
    float* gc;                  /* h floats: hidden bias gradient                          */
    float* gb;                  /* w floats: visible bias gradient                         */
} cuvdia_rbm_cd1_buffers;

CUVDIA_API int cuvdia_rbm_cd1_step_f32(cuvdia_plan* plan, const float* W_vals, const cuvdia_rbm_cd1_buffers* buffers,
                                       int ncols, int batch_global, int mode, int keep_v1p, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Uniform numbers drawn on the device.  CUV binarises an activation against a uniform number that the
 * device draws (rnd_binarize / fill_rnd_uniform, random/random.cu:86-95,139-177; one generator state
 * per thread, so the numbers depend on the launch geometry).  Here the number of element (row, column)
 * is a pure function of (seed, step, which, row, global column): the counter-based generator
 * Philox4x32-10 (Salmon et al., SC 2011) with counter (row / 4, column, which, step) and key = seed,
 * word row % 4 of its output, as the float (word >> 8) * 2^-24 in [0, 1).  A sampling pass can
 * therefore draw its numbers in registers - nothing is read from memory and a host-fed trainer has
 * nothing to upload but its data - every sharding of the batch columns (col0 = global index of the
 * caller's first column) draws what the unsharded run draws, and a CPU restatement gives the same
 * bits (oracle/cuv_host_oracle.c).  step < 2^32, 0 <= which < 65536.
 * ------------------------------------------------------------------------------------------- */
typedef struct cuvdia_draw {
    unsigned long long seed;    /* key of the generator                                      */
    unsigned long long step;    /* distinguishes the steps of a run                          */
    long long col0;             /* global index of the first batch column the call sees      */
} cuvdia_draw;

/* dst[row, col] = that uniform number, rows x ncols, column-major with leading dimension ld
 * (fill_rnd_uniform, random/random.cu:167-177, made reproducible). */
CUVDIA_API int cuvdia_uniform_f32(float* dst, int ld, int rows, int ncols, const cuvdia_draw* draw, int which,
                                  void* stream);

/* act[row, col] = act[row, col] > u ? 1 : 0 in place, u = that uniform number (rnd_binarize,
 * random/random.cu:86-91,139-156). */
CUVDIA_API int cuvdia_rnd_binarize_f32(float* act, int ld, int rows, int ncols, const cuvdia_draw* draw, int which,
                                       void* stream);

/* cuvdia_bias_sigmoid_sample_sum_f32 with the uniform numbers drawn in the kernel instead of read from u:
 * bit for bit what that call gives on u = cuvdia_uniform_f32(draw, which) (rnd_binarize fused into the pass,
 * random/random.cu:139-156). */
CUVDIA_API int cuvdia_bias_sigmoid_draw_sum_f32(float* act, int ld, const float* bias, float* sample, int lds, int units,
                                                int ncols, float* sum_dst, int sum_of_sample, float factNew,
                                                float factOld, int store_act, const cuvdia_draw* draw, int which,
                                                void* stream);

/* cuvdia_rbm_cd1_step_f32 with the hidden (which = 0) and visible (which = 1) samples drawn on the device:
 * buffers->U_h and U_v are not read and may be NULL.  Bit for bit the step on U_h = cuvdia_uniform_f32(draw, 0),
 * U_v = cuvdia_uniform_f32(draw, 1). */
CUVDIA_API int cuvdia_rbm_cd1_step_drawn_f32(cuvdia_plan* plan, const float* W_vals, const cuvdia_rbm_cd1_buffers* buffers,
                                             int ncols, int batch_global, int mode, int keep_v1p,
                                             const cuvdia_draw* draw, void* stream);

/* Sum over the ranks of an NCCL communicator, in place, of the per-rank partial gradients of
 * cuvdia_rbm_cd1_step_f32: the diagonals' value array and the bias gradients, as one collective when
 * bias_grad == G_vals + n_g (one buffer) and as one NCCL group otherwise.  CUV has no multi-GPU path;
 * this is the exchange step of the batch-column sharding.  nccl_comm is an ncclComm_t (the caller's, or
 * one from cuvdia_nccl_comm_create) whose device is current.  NCCL is looked up at run time - the copy
 * already loaded into the process if there is one, else libnccl.so.2 - so this library does not link
 * against it; CUVDIA_ERR_UNSUPPORTED if none can be loaded.  Stream-ordered. */
CUVDIA_API int cuvdia_allreduce_grad(void* nccl_comm, float* G_vals, long long n_g, float* bias_grad, long long n_bias,
                                     void* stream);

/* cuvdia_rbm_cd1_step_f32 and cuvdia_allreduce_grad in one call, with part of the collective hidden under the
 * step's last kernel: when G is a band computed by the tiled kernel and cutting that call in two launches by column
 * tiles costs no wave of blocks, the diagonals the first launch completes (a contiguous slab of G_vals) are summed over
 * the ranks on a side stream of the plan (highest priority) while the second launch computes; the rest of G_vals and
 * the bias gradients follow on `stream`, which then waits for the side stream.  Otherwise it is exactly the two
 * separate calls.  overlap: 0 = never cut (the two separate calls), 1 = cut when it is free, 2 = cut whenever the
 * tiled kernel computes G with at least three column tiles (also with a batch that would otherwise be split: the cut
 * launches are not split).  Results equal those of the two separate calls up to the batch-sum tolerance, and bit for
 * bit when the uncut call would not split the batch (the same sums).  gc and gb should be one array (gb == gc + h), as
 * should G_vals and gc (gc == G_vals + num_dia*stride), for one collective per part.  Every rank must make the same
 * sequence of calls with the same arguments.  No counterpart in CUV. */
CUVDIA_API int cuvdia_rbm_cd1_step_allreduce_f32(cuvdia_plan* plan, const float* W_vals,
                                                 const cuvdia_rbm_cd1_buffers* buffers, int ncols, int batch_global,
                                                 int mode, int keep_v1p, int overlap, void* nccl_comm, void* stream);

/* The same with the samples drawn on the device (see cuvdia_rbm_cd1_step_drawn_f32). */
CUVDIA_API int cuvdia_rbm_cd1_step_drawn_allreduce_f32(cuvdia_plan* plan, const float* W_vals,
                                                       const cuvdia_rbm_cd1_buffers* buffers, int ncols,
                                                       int batch_global, int mode, int keep_v1p, const cuvdia_draw* draw,
                                                       int overlap, void* nccl_comm, void* stream);

/* For callers without a communicator of their own: ncclGetUniqueId on one rank (128 bytes, to be sent
 * to the others by whatever means the application has), then ncclCommInitRank on every rank with its
 * device current (blocking, collective), and ncclCommDestroy. */
CUVDIA_API int cuvdia_nccl_unique_id(char id128[128]);
CUVDIA_API int cuvdia_nccl_comm_create(void** nccl_comm, int nranks, int rank, const char id128[128]);
CUVDIA_API int cuvdia_nccl_comm_destroy(void* nccl_comm);

/* dst = a*x + b*y element-wise over n floats (apply_binary_functor BF_AXPBY,
 * tensor_ops/tensor_ops.hpp:530-655, tensor_ops/functors.hpp:412-433); dst may alias x or y. */
CUVDIA_API int cuvdia_axpby_f32(float* dst, const float* x, const float* y, float a, float b, long long n,
                     void* stream);

/* Gradient step with L2 weight decay over n floats, in place:
 *   W = (-learnrate)*dW + (1 - learnrate*decay)*W
 * (learn_step_weight_decay, tensor_ops/rprop.hpp:117-128, rprop.cu:147-156,331-346; the L1 term
 * `sparsedecay` is commented out in both of the reference's implementations and has no effect there).
 * For a DIA matrix pass its value array and num_dia*stride, as examples/rbm/base.py:72-75 does with
 * the weight matrix and the two bias vectors.  Bit-identical to the host loop. */
CUVDIA_API int cuvdia_learn_step_weight_decay_f32(float* W, const float* dW, long long n, float learnrate,
                                                  float decay, void* stream);

/* The same step with momentum (learn_step_weight_decay_momentum, tensor_ops/rprop.hpp:130-143), with
 * the formula of the reference's device kernel (rprop.cu:158-170):
 *   m = momentum_weight*m - learnrate*(dW + decay*W);   W += m;   momentum = m
 * (the reference's host loop, rprop.cu:356-367, has `dW - decay*W` instead; with decay == 0, the only
 * value its tests use, the two agree). */
CUVDIA_API int cuvdia_learn_step_weight_decay_momentum_f32(float* W, float* momentum, const float* dW, long long n,
                                                           float learnrate, float momentum_weight, float decay,
                                                           void* stream);

/* dst = op(x, y) element-wise over n floats for the float functors of apply_binary_functor the DIA
 * path's callers use (tensor_ops/tensor_ops.hpp:460-492,530-655; functors.hpp:377-433):
 * ADD x+y, SUBTRACT x-y, MULT x*y, AXPY p*x+y, XPBY x+p*y, AXPBY p*x+p2*y.  dst may alias x or y. */
#define CUVDIA_BF_ADD      0
#define CUVDIA_BF_SUBTRACT 1
#define CUVDIA_BF_MULT     2
#define CUVDIA_BF_AXPY     3
#define CUVDIA_BF_XPBY     4
#define CUVDIA_BF_AXPBY    5
CUVDIA_API int cuvdia_binary_f32(float* dst, const float* x, const float* y, int op, float p, float p2,
                                 long long n, void* stream);

/* fill(v, value) and sequence(v) (0, 1, 2, ...) on device tensors (tensor_ops/tensor_ops.hpp:108-122;
 * sequence is thrust::sequence there, tensor_ops.cuh:251-252). */
CUVDIA_API int cuvdia_fill_f32(float* dst, float value, long long n, void* stream);
CUVDIA_API int cuvdia_sequence_f32(float* dst, long long n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CUVDIA_H */
