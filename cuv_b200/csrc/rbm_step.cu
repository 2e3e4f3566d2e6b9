// The sparse-RBM CD-1 step as one C entry point, and the sum of the per-rank gradients over NCCL.
//
// cuvdia_rbm_cd1_step_f32 queues, on one stream and without touching the host in between, the calls
// CUV's RBM trainer makes for one contrastive-divergence step with one Gibbs step
// (examples/rbm/base.py:223-258; upPass/downPass :48-54, gradient accumulation :76-83), with the dense
// weight products replaced by their DIA forms:
//     gb  =  1/B sum_b V0                              reduce_to_col
//     H0p = sigm(W V0 + c),   H0 = H0p > U_h,  gc  =  1/B sum_b H0p       prod 'n' + one element-wise pass
//     V1p = sigm(W^T H0 + b), V1 = V1p > U_v,  gb -=  1/B sum_b V1        prod 't' + one element-wise pass
//     H1p = sigm(W V1 + c),                    gc -=  1/B sum_b H1p       prod 'n' + one element-wise pass
//     G   =  1/B (H0p V0^T)|dia                        densedense_to_dia(1/B, 0)
//     G  += -1/B (H1p V1^T)|dia                        densedense_to_dia(-1/B, 1)
// B is the GLOBAL batch: a rank that holds ncols < B of the batch columns produces partial sums, which
// cuvdia_allreduce_grad completes.  NCCL is looked up at run time (dlopen), so the library has no link-time
// dependency on it and single-GPU users never load it.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "cuvdia_internal.cuh"

namespace cuvdia {

// ---- the few NCCL declarations this file needs (public API of nccl.h, stable across NCCL 2.x) ----------------
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;                 // ncclSuccess == 0
constexpr int kNcclFloat32 = 7;           // ncclFloat32 of ncclDataType_t
constexpr int kNcclSum = 0;               // ncclSum of ncclRedOp_t

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
    bool ok;
};

// The NCCL that is already in the process (e.g. the one a host framework loaded: a communicator handed in by the
// caller belongs to that copy) is preferred; otherwise the system's libnccl.so.2 is loaded.
static const NcclApi* nccl_api() {
    static NcclApi api = {};
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(dlsym(h, "ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GroupStart &&
                 api.GroupEnd && api.GetErrorString;
    });
    return api.ok ? &api : nullptr;
}

static int nccl_fail(const NcclApi* n, ncclResult_t r, const char* what) {
    set_last_error("%s: %s", what, n->GetErrorString(r));
    return CUVDIA_ERR_CUDA;
}

#define CUVDIA_NCCL(n, call)                                            \
    do {                                                                \
        ncclResult_t r__ = (call);                                      \
        if (r__ != 0) return nccl_fail(n, r__, #call);                  \
    } while (0)

static const NcclApi* need_nccl() {
    const NcclApi* n = nccl_api();
    if (!n) {
        const char* why = dlerror();
        set_last_error("libnccl.so.2 could not be loaded (dlopen): %s", why ? why : "a symbol is missing");
    }
    return n;
}

}  // namespace cuvdia

using namespace cuvdia;

extern "C" {

// The step up to and including the first densedense_to_dia (everything but the call that completes G).
static int rbm_step_head(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols, int batch_global,
                         int mode, int keep_v1p, cudaStream_t st, float* inv_out, const cuvdia_draw* draw = nullptr);
static int rbm_step_allreduce(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                              int batch_global, int mode, int keep_v1p, int overlap, void* nccl_comm, void* stream,
                              const cuvdia_draw* draw);

int cuvdia_rbm_cd1_step_f32(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                            int batch_global, int mode, int keep_v1p, void* stream) {
    float inv = 0.f;
    int rc = rbm_step_head(p, W_vals, b, ncols, batch_global, mode, keep_v1p, (cudaStream_t)stream, &inv);
    if (rc) return rc;
    return launch_dd2dia(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols, -inv, 1.f, (cudaStream_t)stream);
}

int cuvdia_rbm_cd1_step_drawn_f32(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                                  int batch_global, int mode, int keep_v1p, const cuvdia_draw* draw, void* stream) {
    CUVDIA_REQUIRE(draw != nullptr);
    float inv = 0.f;
    int rc = rbm_step_head(p, W_vals, b, ncols, batch_global, mode, keep_v1p, (cudaStream_t)stream, &inv, draw);
    if (rc) return rc;
    return launch_dd2dia(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols, -inv, 1.f, (cudaStream_t)stream);
}

static int allreduce_two(const NcclApi* n, ncclComm_t comm, float* G_vals, long long n_g, float* bias_grad, long long n_bias,
                         cudaStream_t st) {
    if (n_g > 0 && n_bias > 0 && bias_grad == G_vals + n_g) {
        // one buffer: one collective
        CUVDIA_NCCL(n, n->AllReduce(G_vals, G_vals, (size_t)(n_g + n_bias), kNcclFloat32, kNcclSum, comm, st));
        return CUVDIA_OK;
    }
    CUVDIA_NCCL(n, n->GroupStart());
    ncclResult_t r1 = n_g > 0 ? n->AllReduce(G_vals, G_vals, (size_t)n_g, kNcclFloat32, kNcclSum, comm, st) : 0;
    ncclResult_t r2 = n_bias > 0 ? n->AllReduce(bias_grad, bias_grad, (size_t)n_bias, kNcclFloat32, kNcclSum, comm, st) : 0;
    ncclResult_t r3 = n->GroupEnd();
    if (r1) return nccl_fail(n, r1, "ncclAllReduce(G)");
    if (r2) return nccl_fail(n, r2, "ncclAllReduce(bias gradients)");
    if (r3) return nccl_fail(n, r3, "ncclGroupEnd");
    return CUVDIA_OK;
}

int cuvdia_rbm_cd1_step_allreduce_f32(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                                      int batch_global, int mode, int keep_v1p, int overlap, void* nccl_comm,
                                      void* stream) {
    return rbm_step_allreduce(p, W_vals, b, ncols, batch_global, mode, keep_v1p, overlap, nccl_comm, stream, nullptr);
}

int cuvdia_rbm_cd1_step_drawn_allreduce_f32(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                                            int batch_global, int mode, int keep_v1p, const cuvdia_draw* draw, int overlap,
                                            void* nccl_comm, void* stream) {
    CUVDIA_REQUIRE(draw != nullptr);
    return rbm_step_allreduce(p, W_vals, b, ncols, batch_global, mode, keep_v1p, overlap, nccl_comm, stream, draw);
}

static int rbm_step_allreduce(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols,
                              int batch_global, int mode, int keep_v1p, int overlap, void* nccl_comm, void* stream,
                              const cuvdia_draw* draw) {
    CUVDIA_REQUIRE(nccl_comm != nullptr);
    CUVDIA_REQUIRE(overlap >= 0 && overlap <= 2);
    const NcclApi* n = need_nccl();
    if (!n) return CUVDIA_ERR_UNSUPPORTED;
    ncclComm_t comm = (ncclComm_t)nccl_comm;
    cudaStream_t st = (cudaStream_t)stream;
    float inv = 0.f;
    int rc = rbm_step_head(p, W_vals, b, ncols, batch_global, mode, keep_v1p, st, &inv, draw);
    if (rc) return rc;
    const long long n_g = (long long)p->nd * p->stride, n_bias = (long long)p->h + p->w;
    float* bias = b->gc;                                  // gc then gb: one array when gb follows gc
    const bool bias_one = b->gb == b->gc + p->h;
    // Cut the call that completes G in two launches by column tiles when that costs no wave of blocks: the diagonals
    // the first launch completes are summed over the ranks on a side stream while the second launch computes.
    int first_diagonals = 0;
    const int cut = (overlap > 0 && bias_one && dd2dia_band_applicable(p, b->H1p, p->h, b->V1, p->w, ncols) &&
                     !dd2dia_stream_applicable(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols) &&
                     (overlap == 2 || dd2dia_band_nsplit(p, ncols) == 1))
                        ? dd2dia_band_cut(p, ncols, &first_diagonals, overlap == 2) : 0;
    if (cut <= 0) {
        rc = launch_dd2dia(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols, -inv, 1.f, st);
        if (rc) return rc;
        if (bias_one) return allreduce_two(n, comm, b->G_vals, n_g, bias, n_bias, st);
        rc = allreduce_two(n, comm, b->G_vals, n_g, b->gc, p->h, st);
        if (rc) return rc;
        CUVDIA_NCCL(n, n->AllReduce(b->gb, b->gb, (size_t)p->w, kNcclFloat32, kNcclSum, comm, st));
        return CUVDIA_OK;
    }
    if (!p->side_stream) {
        int lo = 0, hi = 0;
        CUVDIA_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));       // hi = numerically lowest = highest priority
        CUVDIA_CUDA(cudaStreamCreateWithPriority(&p->side_stream, cudaStreamNonBlocking, hi));
        CUVDIA_CUDA(cudaEventCreateWithFlags(&p->ev_first, cudaEventDisableTiming));
        CUVDIA_CUDA(cudaEventCreateWithFlags(&p->ev_side, cudaEventDisableTiming));
    }
    rc = launch_dd2dia_band_range(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols, -inv, 1.f, 0, cut, st);
    if (rc) return rc;
    CUVDIA_CUDA(cudaEventRecord(p->ev_first, st));
    CUVDIA_CUDA(cudaStreamWaitEvent(p->side_stream, p->ev_first, 0));
    const long long n_first = (long long)first_diagonals * p->stride;
    CUVDIA_NCCL(n, n->AllReduce(b->G_vals, b->G_vals, (size_t)n_first, kNcclFloat32, kNcclSum, comm, p->side_stream));
    rc = launch_dd2dia_band_range(p, b->G_vals, b->H1p, p->h, b->V1, p->w, ncols, -inv, 1.f, cut, -1, st);
    if (rc) return rc;
    // the rest of the diagonals and, behind them in the same buffer or on its own, the bias gradients
    const bool tail_one = bias == b->G_vals + n_g;
    CUVDIA_NCCL(n, n->AllReduce(b->G_vals + n_first, b->G_vals + n_first, (size_t)(n_g - n_first + (tail_one ? n_bias : 0)),
                                kNcclFloat32, kNcclSum, comm, st));
    if (!tail_one) CUVDIA_NCCL(n, n->AllReduce(bias, bias, (size_t)n_bias, kNcclFloat32, kNcclSum, comm, st));
    CUVDIA_CUDA(cudaEventRecord(p->ev_side, p->side_stream));
    CUVDIA_CUDA(cudaStreamWaitEvent(st, p->ev_side, 0));
    return CUVDIA_OK;
}

static int rbm_step_head(cuvdia_plan* p, const float* W_vals, const cuvdia_rbm_cd1_buffers* b, int ncols, int batch_global,
                         int mode, int keep_v1p, cudaStream_t st, float* inv_out, const cuvdia_draw* draw) {
    CUVDIA_REQUIRE(p != nullptr && W_vals != nullptr && b != nullptr);
    CUVDIA_REQUIRE(p->rf == 1);                        // the trainer's weight matrix (row factors belong to other layers)
    CUVDIA_REQUIRE(ncols > 0 && batch_global >= ncols);
    CUVDIA_REQUIRE(mode == CUVDIA_MODE_EXACT || mode == CUVDIA_MODE_FAST);
    CUVDIA_REQUIRE(b->V0 != nullptr);
    if (draw) { CUVDIA_REQUIRE(draw->col0 >= 0 && draw->step < (1ull << 32)); }
    else      { CUVDIA_REQUIRE(b->U_h && b->U_v); }
    // draw 0: the hidden sample, draw 1: the visible sample (U_h and U_v are not read)
    DrawParams d_h = {}, d_v = {};
    if (draw) { d_h = make_draw(draw, 0); d_v = make_draw(draw, 1); }
    CUVDIA_REQUIRE(b->H0p && b->H0 && b->V1p && b->V1 && b->H1p);
    CUVDIA_REQUIRE(b->G_vals && b->gc && b->gb);
    int dev = -1;
    CUVDIA_REQUIRE(cudaGetDevice(&dev) == cudaSuccess && dev == p->device);
    const int hid = p->h, vis = p->w;
    const float inv = (float)(1.0 / (double)batch_global);
    *inv_out = inv;
    int rc;
#define STEP(call) do { rc = (call); if (rc) return rc; } while (0)
    STEP(launch_reduce(b->gb, b->V0, vis, ncols, true, CUVDIA_RF_ADD, inv, 0.f, st));
    STEP(launch_prod(p, W_vals, b->V0, vis, b->H0p, hid, ncols, false, 1.f, 0.f, mode, nullptr, st));
    STEP(launch_bias_sigmoid_sample_sum(b->H0p, hid, b->c_hid, draw ? nullptr : b->U_h, hid, b->H0, hid, hid, ncols, b->gc, 0, inv,
                                        0.f, 1, st, draw ? &d_h : nullptr));
    STEP(launch_prod(p, W_vals, b->H0, hid, b->V1p, vis, ncols, true, 1.f, 0.f, mode, nullptr, st));
    STEP(launch_bias_sigmoid_sample_sum(b->V1p, vis, b->b_vis, draw ? nullptr : b->U_v, vis, b->V1, vis, vis, ncols, b->gb, 1, -inv,
                                        1.f, keep_v1p ? 1 : 0, st, draw ? &d_v : nullptr));
    STEP(launch_prod(p, W_vals, b->V1, vis, b->H1p, hid, ncols, false, 1.f, 0.f, mode, nullptr, st));
    STEP(launch_bias_sigmoid_sample_sum(b->H1p, hid, b->c_hid, nullptr, 0, nullptr, 0, hid, ncols, b->gc, 0, -inv, 1.f, 1, st));
    STEP(launch_dd2dia(p, b->G_vals, b->H0p, hid, b->V0, vis, ncols, inv, 0.f, st));
#undef STEP
    return CUVDIA_OK;
}

int cuvdia_allreduce_grad(void* nccl_comm, float* G_vals, long long n_g, float* bias_grad, long long n_bias,
                          void* stream) {
    CUVDIA_REQUIRE(nccl_comm != nullptr);
    CUVDIA_REQUIRE(n_g >= 0 && n_bias >= 0);
    CUVDIA_REQUIRE(n_g == 0 || G_vals != nullptr);
    CUVDIA_REQUIRE(n_bias == 0 || bias_grad != nullptr);
    const NcclApi* n = need_nccl();
    if (!n) return CUVDIA_ERR_UNSUPPORTED;
    return allreduce_two(n, (ncclComm_t)nccl_comm, G_vals, n_g, bias_grad, n_bias, (cudaStream_t)stream);
}

int cuvdia_nccl_unique_id(char id128[128]) {
    CUVDIA_REQUIRE(id128 != nullptr);
    const NcclApi* n = need_nccl();
    if (!n) return CUVDIA_ERR_UNSUPPORTED;
    ncclUniqueId id;
    CUVDIA_NCCL(n, n->GetUniqueId(&id));
    memcpy(id128, id.internal, 128);
    return CUVDIA_OK;
}

int cuvdia_nccl_comm_create(void** comm, int nranks, int rank, const char id128[128]) {
    CUVDIA_REQUIRE(comm != nullptr && id128 != nullptr);
    CUVDIA_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks);
    *comm = nullptr;
    const NcclApi* n = need_nccl();
    if (!n) return CUVDIA_ERR_UNSUPPORTED;
    ncclUniqueId id;
    memcpy(id.internal, id128, 128);
    ncclComm_t c = nullptr;
    CUVDIA_NCCL(n, n->CommInitRank(&c, nranks, id, rank));
    *comm = c;
    return CUVDIA_OK;
}

int cuvdia_nccl_comm_destroy(void* comm) {
    if (!comm) return CUVDIA_OK;
    const NcclApi* n = need_nccl();
    if (!n) return CUVDIA_ERR_UNSUPPORTED;
    CUVDIA_NCCL(n, n->CommDestroy((ncclComm_t)comm));
    return CUVDIA_OK;
}

}  // extern "C"
