// extern "C" layer of libcuvdia.so: argument checks (CUV's cuvAssert preconditions turned into
// error codes), the plan object, error strings and the per-stream workspace.
#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <set>

#include "cuvdia_internal.cuh"

namespace cuvdia {

static thread_local std::string t_last_error;
std::atomic<unsigned long long> g_launches{0};

void set_last_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
}

int cuda_fail(cudaError_t e, const char* what) {
    set_last_error("%s: %s", what, cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? CUVDIA_ERR_NOMEM : CUVDIA_ERR_CUDA;
}

int check_launch(const char* kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, kernel);
    return CUVDIA_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

struct Workspace { void* ptr = nullptr; size_t bytes = 0; };
static std::mutex g_ws_mutex;
static std::map<std::pair<int, cudaStream_t>, Workspace> g_ws;

int get_workspace(cudaStream_t stream, size_t bytes, void** ptr) {
    int dev = 0;
    CUVDIA_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    Workspace& ws = g_ws[std::make_pair(dev, stream)];
    if (ws.bytes < bytes) {
        if (ws.ptr) {
            // the old buffer may still be in use by work queued on this stream
            CUVDIA_CUDA(cudaStreamSynchronize(stream));
            CUVDIA_CUDA(cudaFree(ws.ptr));
            ws.ptr = nullptr; ws.bytes = 0;
        }
        size_t want = std::max(bytes, (size_t)1 << 20);
        CUVDIA_CUDA(cudaMalloc(&ws.ptr, want));
        ws.bytes = want;
    }
    *ptr = ws.ptr;
    return CUVDIA_OK;
}

int release_workspaces() {
    CUVDIA_CUDA(cudaDeviceSynchronize());
    int dev = 0;
    CUVDIA_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    for (auto it = g_ws.begin(); it != g_ws.end();) {
        if (it->first.first == dev) {
            if (it->second.ptr) cudaFree(it->second.ptr);
            it = g_ws.erase(it);
        } else ++it;
    }
    return CUVDIA_OK;
}

}  // namespace cuvdia

using namespace cuvdia;

// A plan's device arrays live on the device that was current when it was created.
static bool plan_on_current_device(const cuvdia_plan* p) {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess && dev == p->device;
}

extern "C" {

const char* cuvdia_error_string(int code) {
    switch (code) {
        case CUVDIA_OK: return "success";
        case CUVDIA_ERR_INVALID: return "precondition failed (invalid argument)";
        case CUVDIA_ERR_CUDA: return "CUDA runtime error";
        case CUVDIA_ERR_UNSUPPORTED: return "not supported";
        case CUVDIA_ERR_NOMEM: return "out of memory";
        default: return "unknown cuvdia error code";
    }
}

const char* cuvdia_last_error_message(void) { return t_last_error.c_str(); }

int cuvdia_release_workspaces(void) { return release_workspaces(); }

unsigned long long cuvdia_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int cuvdia_plan_create(cuvdia_plan** out, int h, int w, int num_dia, int stride, int row_fact,
                       const int* offsets_host) {
    CUVDIA_REQUIRE(out != nullptr);
    *out = nullptr;
    CUVDIA_REQUIRE(h > 0 && w > 0);
    CUVDIA_REQUIRE(num_dia > 0);
    CUVDIA_REQUIRE(row_fact > 0);                       // basics/dia_matrix.hpp:106
    CUVDIA_REQUIRE(stride >= h);                        // cells are indexed by row (dia_matrix.hpp:234,242)
    CUVDIA_REQUIRE(offsets_host != nullptr);
    CUVDIA_REQUIRE((long long)num_dia * (long long)stride <= 2147483647LL);   // basics/tensor.hpp:209-213
    cuvdia_plan* p = new (std::nothrow) cuvdia_plan();
    if (!p) { set_last_error("host allocation failed"); return CUVDIA_ERR_NOMEM; }
    p->h = h; p->w = w; p->nd = num_dia; p->stride = stride; p->rf = row_fact;
    p->offsets.assign(offsets_host, offsets_host + num_dia);
    p->d_offsets = nullptr; p->scratch = nullptr; p->scratch_floats = 0; p->d_status = nullptr; p->d_passes = nullptr; p->d_sorted = nullptr; p->d_witems = nullptr;
    p->side_stream = nullptr; p->ev_first = nullptr; p->ev_side = nullptr;
    p->is_band = true;
    for (int k = 1; k < num_dia; k++) if (p->offsets[k] != p->offsets[0] + k) { p->is_band = false; break; }
    p->band_lo = p->offsets[0];
    p->off_min = *std::min_element(p->offsets.begin(), p->offsets.end());
    p->off_max = *std::max_element(p->offsets.begin(), p->offsets.end());
    p->nnz = 0;
    for (int k = 0; k < num_dia; k++) {                 // matrix_ops/spmv.cu:185-189
        long long o = p->offsets[k];
        long long rs = (long long)row_fact * std::max(0LL, -o), js = std::max(0LL, o);
        long long n = std::min((long long)h - rs, (long long)row_fact * ((long long)w - js));
        if (n > 0) p->nnz += n;
    }
    // runs of consecutive diagonal numbers, cut into passes of at most 8
    std::vector<int> passes;
    for (int k = 0; k < num_dia;) {
        int len = 1;
        while (k + len < num_dia && p->offsets[k + len] == p->offsets[k + len - 1] + 1) len++;
        for (int s = 0; s < len; s += 8) {
            passes.push_back(k + s); passes.push_back(p->offsets[k] + s); passes.push_back(std::min(8, len - s));
            passes.push_back(0);
        }
        k += len;
    }
    p->npass = (int)(passes.size() / 4);
    p->is_runs = row_fact == 1 && num_dia >= 8 && (long long)p->npass * 4 <= num_dia;
    p->d_passes = nullptr;
    // diagonals in ascending order of their offsets (stable, so repeated numbers keep their storage order)
    std::vector<int> order(num_dia);
    for (int k = 0; k < num_dia; k++) order[k] = k;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return p->offsets[a] < p->offsets[b]; });
    std::vector<int> sorted(2 * (size_t)num_dia);
    for (int k = 0; k < num_dia; k++) { sorted[k] = order[k]; sorted[num_dia + k] = p->offsets[order[k]]; }
    std::vector<int> witems;
    window_items(h, w, num_dia, row_fact, sorted.data() + num_dia, &witems);
    p->n_witems = (int)(witems.size() / 3);
    p->witem_diagonals = 0;
    for (int t = 0; t < p->n_witems; t++) p->witem_diagonals += witems[3 * t + 2];
    p->d_sorted = nullptr; p->d_witems = nullptr;
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaMalloc(&p->d_offsets, sizeof(int) * (size_t)num_dia);
    if (e == cudaSuccess) e = cudaMalloc(&p->d_sorted, sizeof(int) * sorted.size());
    if (e == cudaSuccess)
        e = cudaMemcpy(p->d_sorted, sorted.data(), sizeof(int) * sorted.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess && p->n_witems > 0) {
        e = cudaMalloc(&p->d_witems, sizeof(int) * witems.size());
        if (e == cudaSuccess)
            e = cudaMemcpy(p->d_witems, witems.data(), sizeof(int) * witems.size(), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess && p->is_runs) {
        e = cudaMalloc(&p->d_passes, sizeof(int) * passes.size());
        if (e == cudaSuccess)
            e = cudaMemcpy(p->d_passes, passes.data(), sizeof(int) * passes.size(), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess)
        e = cudaMemcpy(p->d_offsets, p->offsets.data(), sizeof(int) * (size_t)num_dia, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&p->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->d_status, 0, sizeof(int));
    if (e != cudaSuccess) {
        if (p->d_offsets) cudaFree(p->d_offsets);
        if (p->d_status) cudaFree(p->d_status);
        if (p->d_passes) cudaFree(p->d_passes);
        if (p->d_sorted) cudaFree(p->d_sorted);
        if (p->d_witems) cudaFree(p->d_witems);
        delete p;
        return cuda_fail(e, "cuvdia_plan_create");
    }
    *out = p;
    return CUVDIA_OK;
}

int cuvdia_plan_destroy(cuvdia_plan* p) {
    if (!p) return CUVDIA_OK;
    if (p->d_offsets) cudaFree(p->d_offsets);
    if (p->scratch) cudaFree(p->scratch);
    if (p->d_status) cudaFree(p->d_status);
    if (p->d_passes) cudaFree(p->d_passes);
    if (p->d_sorted) cudaFree(p->d_sorted);
    if (p->d_witems) cudaFree(p->d_witems);
    if (p->ev_first) cudaEventDestroy(p->ev_first);
    if (p->ev_side) cudaEventDestroy(p->ev_side);
    if (p->side_stream) cudaStreamDestroy(p->side_stream);
    delete p;
    return CUVDIA_OK;
}

int cuvdia_plan_info(const cuvdia_plan* p, int* is_band, long long* nnz) {
    CUVDIA_REQUIRE(p != nullptr);
    if (is_band) *is_band = p->is_band ? 1 : 0;
    if (nnz) *nnz = p->nnz;
    return CUVDIA_OK;
}

int cuvdia_plan_status(const cuvdia_plan* p, int* status) {
    CUVDIA_REQUIRE(p != nullptr && status != nullptr);
    CUVDIA_CUDA(cudaMemcpy(status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    return CUVDIA_OK;
}

const int* cuvdia_plan_offsets_device(const cuvdia_plan* p) { return p ? p->d_offsets : nullptr; }

int cuvdia_plan_status_clear(cuvdia_plan* p, void* stream) {
    CUVDIA_REQUIRE(p != nullptr);
    CUVDIA_REQUIRE(plan_on_current_device(p));
    CUVDIA_CUDA(cudaMemsetAsync(p->d_status, 0, sizeof(int), (cudaStream_t)stream));
    return CUVDIA_OK;
}

int cuvdia_selftest_bounded_wait(cuvdia_plan* p, unsigned max_polls, void* stream) {
    CUVDIA_REQUIRE(p != nullptr);
    CUVDIA_REQUIRE(max_polls >= 1 && max_polls <= (1u << 20));       // a self-test, not a stress test
    CUVDIA_REQUIRE(plan_on_current_device(p));
    return launch_selftest_wait(p->d_status, max_polls, (cudaStream_t)stream);
}

int cuvdia_prod_f32(const cuvdia_plan* p, const float* A_vals, const float* B, int ldb, float* C, int ldc,
                    int ncols, char transA, char transB, float factAB, float factC, int mode, void* stream) {
    CUVDIA_REQUIRE(p != nullptr);
    CUVDIA_REQUIRE(transB == 'n');                       // matrix_ops/spmv.cu:213,231
    CUVDIA_REQUIRE(transA == 'n' || transA == 't');      // make_spmv_header.pl:121-123
    CUVDIA_REQUIRE(C != nullptr);                        // spmv.cu:233
    CUVDIA_REQUIRE(A_vals != nullptr);                   // spmv.cu:234
    CUVDIA_REQUIRE(B != nullptr);                        // spmv.cu:235
    CUVDIA_REQUIRE(ncols >= 0);
    CUVDIA_REQUIRE(mode == CUVDIA_MODE_EXACT || mode == CUVDIA_MODE_FAST);
    CUVDIA_REQUIRE(plan_on_current_device(p));
    const bool trans = transA == 't';
    const int rows_b = trans ? p->h : p->w, rows_c = trans ? p->w : p->h;
    CUVDIA_REQUIRE(ldb >= rows_b);                       // spmv.cu:159,180 (operand heights)
    CUVDIA_REQUIRE(ldc >= rows_c);                       // spmv.cu:160,181,236-240
    if (ncols == 0) return CUVDIA_OK;
    return launch_prod(p, A_vals, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, nullptr, (cudaStream_t)stream);
}

int cuvdia_prod_bias_sigmoid_sample_f32(const cuvdia_plan* p, const float* A_vals, const float* B, int ldb, float* C,
                                        int ldc, int ncols, char transA, float factAB, float factC, int mode,
                                        const float* bias, const float* u, int ldu, float* sample, int lds,
                                        void* stream) {
    CUVDIA_REQUIRE(p != nullptr);
    CUVDIA_REQUIRE(transA == 'n' || transA == 't');
    CUVDIA_REQUIRE(C != nullptr && A_vals != nullptr && B != nullptr);
    CUVDIA_REQUIRE(ncols >= 0);
    CUVDIA_REQUIRE(mode == CUVDIA_MODE_EXACT || mode == CUVDIA_MODE_FAST);
    CUVDIA_REQUIRE(plan_on_current_device(p));
    const bool trans = transA == 't';
    const int rows_b = trans ? p->h : p->w, rows_c = trans ? p->w : p->h;
    CUVDIA_REQUIRE(ldb >= rows_b);
    CUVDIA_REQUIRE(ldc >= rows_c);
    CUVDIA_REQUIRE((u == nullptr) == (sample == nullptr));
    if (u) { CUVDIA_REQUIRE(ldu >= rows_c); CUVDIA_REQUIRE(lds >= rows_c); }
    if (ncols == 0) return CUVDIA_OK;
    ProdEpilogue ep = {bias, u, ldu, sample, lds};
    return launch_prod(p, A_vals, B, ldb, C, ldc, ncols, trans, factAB, factC, mode, &ep, (cudaStream_t)stream);
}

int cuvdia_dd2dia_f32(cuvdia_plan* p, float* C_vals, const float* A, int lda, const float* B, int ldb, int ncols,
                      float factAB, float factC, void* stream) {
    CUVDIA_REQUIRE(p != nullptr);
    CUVDIA_REQUIRE(C_vals != nullptr);
    CUVDIA_REQUIRE(A != nullptr && B != nullptr);
    CUVDIA_REQUIRE(ncols >= 0);
    CUVDIA_REQUIRE(lda >= p->h);                         // densedense_to_sparse.cu:215,277
    CUVDIA_REQUIRE(ldb >= p->w);                         // densedense_to_sparse.cu:214,276
    CUVDIA_REQUIRE(p->h % p->rf == 0);                   // densedense_to_sparse.cu:244-249 overruns otherwise
    CUVDIA_REQUIRE(plan_on_current_device(p));
    return launch_dd2dia(p, C_vals, A, lda, B, ldb, ncols, factAB, factC, (cudaStream_t)stream);
}

int cuvdia_reduce_f32(float* dst, const float* src, long long n_contig, long long n_strided, int over_strided,
                      int functor, float factNew, float factOld, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr);
    CUVDIA_REQUIRE(src != nullptr);                      // matrix_ops_reduce.cu:160,192
    CUVDIA_REQUIRE(n_contig > 0 && n_strided > 0);
    CUVDIA_REQUIRE(n_contig * n_strided <= 2147483647LL);
    CUVDIA_REQUIRE(functor >= CUVDIA_RF_ADD && functor <= CUVDIA_RF_ADDEXP);
    if (functor == CUVDIA_RF_MEAN) {                     // matrix_ops_reduce.cu:309-310
        CUVDIA_REQUIRE(factNew == 1.f);
        CUVDIA_REQUIRE(factOld == 0.f);
    }
    return launch_reduce(dst, src, n_contig, n_strided, over_strided != 0, functor, factNew, factOld,
                         (cudaStream_t)stream);
}

int cuvdia_avg_diagonals_f32(const cuvdia_plan* p, const float* A_vals, float* dst, void* stream) {
    CUVDIA_REQUIRE(p != nullptr && A_vals != nullptr && dst != nullptr);
    CUVDIA_REQUIRE(p->rf == 1);                          // matrix_ops/diagonals.cu:28
    CUVDIA_REQUIRE(plan_on_current_device(p));
    return launch_avg_diagonals(p, A_vals, dst, (cudaStream_t)stream);
}

int cuvdia_reduce(void* dst, int dst_type, const void* src, int src_type, long long n_contig, long long n_strided,
                  int over_strided, int functor, float factNew, float factOld, void* stream) {
    if (dst_type == CUVDIA_T_F32 && src_type == CUVDIA_T_F32)
        return cuvdia_reduce_f32((float*)dst, (const float*)src, n_contig, n_strided, over_strided, functor, factNew,
                                 factOld, stream);
    CUVDIA_REQUIRE(dst != nullptr);
    CUVDIA_REQUIRE(src != nullptr);                      // matrix_ops_reduce.cu:160,192
    CUVDIA_REQUIRE(n_contig > 0 && n_strided > 0);
    CUVDIA_REQUIRE(n_contig * n_strided <= 2147483647LL);
    CUVDIA_REQUIRE(functor >= CUVDIA_RF_ADD && functor <= CUVDIA_RF_ADDEXP);
    if (functor == CUVDIA_RF_MEAN) {                     // matrix_ops_reduce.cu:309-310
        CUVDIA_REQUIRE(factNew == 1.f);
        CUVDIA_REQUIRE(factOld == 0.f);
    }
    return launch_reduce_typed(dst, dst_type, src, src_type, n_contig, n_strided, over_strided != 0, functor, factNew,
                               factOld, (cudaStream_t)stream);
}

int cuvdia_bias_sigmoid_sample_f32(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                                   int lds, int units, int ncols, void* stream) {
    CUVDIA_REQUIRE(act != nullptr);
    CUVDIA_REQUIRE(units > 0 && ncols >= 0);
    CUVDIA_REQUIRE(ld >= units);
    CUVDIA_REQUIRE((u == nullptr) == (sample == nullptr));
    if (u) { CUVDIA_REQUIRE(ldu >= units); CUVDIA_REQUIRE(lds >= units); }
    if (ncols == 0) return CUVDIA_OK;
    return launch_bias_sigmoid_sample(act, ld, bias, u, ldu, sample, lds, units, ncols, (cudaStream_t)stream);
}

int cuvdia_bias_sigmoid_sample_sum_f32(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                                       int lds, int units, int ncols, float* sum_dst, int sum_of_sample, float factNew,
                                       float factOld, int store_act, void* stream) {
    CUVDIA_REQUIRE(act != nullptr);
    CUVDIA_REQUIRE(sum_dst != nullptr);
    CUVDIA_REQUIRE(units > 0 && ncols > 0);
    CUVDIA_REQUIRE(ld >= units);
    CUVDIA_REQUIRE((u == nullptr) == (sample == nullptr));
    if (u) { CUVDIA_REQUIRE(ldu >= units); CUVDIA_REQUIRE(lds >= units); }
    CUVDIA_REQUIRE(!sum_of_sample || sample != nullptr);
    CUVDIA_REQUIRE(store_act || sample != nullptr);      // something must be produced besides the sum
    return launch_bias_sigmoid_sample_sum(act, ld, bias, u, ldu, sample, lds, units, ncols, sum_dst, sum_of_sample ? 1 : 0,
                                          factNew, factOld, store_act ? 1 : 0, (cudaStream_t)stream);
}

int cuvdia_uniform_f32(float* dst, int ld, int rows, int ncols, const cuvdia_draw* draw, int which, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr && draw != nullptr);
    CUVDIA_REQUIRE(rows > 0 && ncols >= 0 && ld >= rows);
    CUVDIA_REQUIRE(which >= 0 && which < 65536);
    CUVDIA_REQUIRE(draw->col0 >= 0 && draw->step < (1ull << 32));
    if (ncols == 0) return CUVDIA_OK;
    return launch_uniform(dst, ld, rows, ncols, make_draw(draw, (unsigned)which), (cudaStream_t)stream);
}

int cuvdia_rnd_binarize_f32(float* act, int ld, int rows, int ncols, const cuvdia_draw* draw, int which, void* stream) {
    CUVDIA_REQUIRE(act != nullptr && draw != nullptr);
    CUVDIA_REQUIRE(rows > 0 && ncols >= 0 && ld >= rows);
    CUVDIA_REQUIRE(which >= 0 && which < 65536);
    CUVDIA_REQUIRE(draw->col0 >= 0 && draw->step < (1ull << 32));
    if (ncols == 0) return CUVDIA_OK;
    return launch_binarize(act, ld, rows, ncols, make_draw(draw, (unsigned)which), (cudaStream_t)stream);
}

int cuvdia_bias_sigmoid_draw_sum_f32(float* act, int ld, const float* bias, float* sample, int lds, int units, int ncols,
                                     float* sum_dst, int sum_of_sample, float factNew, float factOld, int store_act,
                                     const cuvdia_draw* draw, int which, void* stream) {
    CUVDIA_REQUIRE(act != nullptr && sample != nullptr && sum_dst != nullptr && draw != nullptr);
    CUVDIA_REQUIRE(units > 0 && ncols > 0);
    CUVDIA_REQUIRE(ld >= units && lds >= units);
    CUVDIA_REQUIRE(which >= 0 && which < 65536);
    CUVDIA_REQUIRE(draw->col0 >= 0 && draw->step < (1ull << 32));
    const DrawParams dp = make_draw(draw, (unsigned)which);
    return launch_bias_sigmoid_sample_sum(act, ld, bias, nullptr, 0, sample, lds, units, ncols, sum_dst, sum_of_sample ? 1 : 0,
                                          factNew, factOld, store_act ? 1 : 0, (cudaStream_t)stream, &dp);
}

int cuvdia_axpby_f32(float* dst, const float* x, const float* y, float a, float b, long long n, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr && x != nullptr && y != nullptr);
    CUVDIA_REQUIRE(n >= 0);
    if (n == 0) return CUVDIA_OK;
    return launch_axpby(dst, x, y, a, b, n, (cudaStream_t)stream);
}

int cuvdia_learn_step_weight_decay_f32(float* W, const float* dW, long long n, float learnrate, float decay,
                                       void* stream) {
    CUVDIA_REQUIRE(W != nullptr && dW != nullptr);
    CUVDIA_REQUIRE(n >= 0);
    if (n == 0) return CUVDIA_OK;
    // the factors are formed in float exactly as the reference forms them (tensor_ops/rprop.cu:345)
    const float alpha = -learnrate;
    const float beta = 1.f - learnrate * decay;
    return launch_learn_step(W, nullptr, dW, alpha, beta, 0.f, n, (cudaStream_t)stream);
}

int cuvdia_learn_step_weight_decay_momentum_f32(float* W, float* momentum, const float* dW, long long n,
                                                float learnrate, float momentum_weight, float decay, void* stream) {
    CUVDIA_REQUIRE(W != nullptr && dW != nullptr && momentum != nullptr);
    CUVDIA_REQUIRE(n >= 0);
    if (n == 0) return CUVDIA_OK;
    return launch_learn_step(W, momentum, dW, learnrate, momentum_weight, decay, n, (cudaStream_t)stream);
}

int cuvdia_binary_f32(float* dst, const float* x, const float* y, int op, float p, float p2, long long n, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr && x != nullptr && y != nullptr);
    CUVDIA_REQUIRE(op >= CUVDIA_BF_ADD && op <= CUVDIA_BF_AXPBY);
    CUVDIA_REQUIRE(n >= 0);
    if (n == 0) return CUVDIA_OK;
    return launch_binary(dst, x, y, op, p, p2, n, (cudaStream_t)stream);
}

int cuvdia_fill_f32(float* dst, float value, long long n, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr && n >= 0);
    if (n == 0) return CUVDIA_OK;
    return launch_fill(dst, value, 0, n, (cudaStream_t)stream);
}

int cuvdia_sequence_f32(float* dst, long long n, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr && n >= 0);
    if (n == 0) return CUVDIA_OK;
    return launch_fill(dst, 0.f, 1, n, (cudaStream_t)stream);
}

}  // extern "C"
