// C++ tests of the CUV surface over libcuvdia.so.  They follow CUV's own tests of this path - same
// fixtures, same "device object vs host object of the same template" pattern:
//   src/tests/spmv.cpp:49-143, src/tests/densedense_to_dia.cpp:50-197, src/tests/dia_mat.cpp:48-132,
//   src/tests/convert.cpp:110-129, src/tests/matrix_op.cpp:80-105,574-628,858-924, src/tests/optimize.cpp:59-121.
// The host halves come from the CPU oracle (oracle/cuv_host_reference.hpp).  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "cuv.hpp"
#include "cuv_host_reference.hpp"

using namespace cuv;

static int g_fail = 0, g_checks = 0;
#define CHECK(cond) do { g_checks++; if (!(cond)) { g_fail++; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } } while (0)

// MAT_CMP of tools/cuv_test.hpp:39-57: element-wise closeness in PERCENT
template <class A, class B> static void mat_cmp(const A& x, const B& y, double percent, const char* what) {
    int bad = 0;
    for (unsigned i = 0; i < x.shape()[0]; i++)
        for (unsigned j = 0; j < x.shape()[1]; j++) {
            const double a = (float)x(i, j), b = (float)y(i, j);
            const double tol = percent * 0.01 * std::max(std::fabs(a), std::fabs(b));
            if (!(std::fabs(a - b) <= tol)) bad++;
        }
    g_checks++;
    if (bad) { g_fail++; std::printf("FAILED %s: %d elements differ by more than %g%%\n", what, bad, percent); }
}
template <class A, class B> static void mat_eq(const A& x, const B& y, const char* what) { mat_cmp(x, y, 0.0, what); }

// ---- spmv.cpp -----------------------------------------------------------------------------------------------
static void test_spmv() {
    const int n = 32, m = 16, k = 6, rf = 1;
    dia_matrix<float, host_memory_space> A(n, m, 7, std::max(n, m), rf);
    tensor<float, host_memory_space, column_major> B(m, k), C(n, k);
    std::vector<int> off;
    for (int i = -A.num_dia() / 2; i <= A.num_dia() / 2; i++) off.push_back(i);
    A.set_offsets(off);
    sequence(A.vec()); sequence(C); sequence(B);
    dia_matrix<float, dev_memory_space> A2(n, m, A.num_dia(), A.stride(), rf);
    convert(A2, A);
    {   // spmv_dev_correctness_trans (:103-115)
        tensor<float, dev_memory_space, column_major> C2(C.shape()), B2(B.shape());
        convert(C2, C); convert(B2, B);
        prod(B, A, C, 't', 'n');
        prod(B2, A2, C2, 't', 'n');
        mat_eq(B, B2, "spmv_dev_correctness_trans");       // exact arithmetic: identical, not just within 0.1 %
    }
    {   // spmv_dev_correctness (:116-129)
        sequence(B); sequence(C);
        tensor<float, dev_memory_space, column_major> C2(C.shape()), B2(B.shape());
        convert(C2, C); convert(B2, B);
        prod(C, A, B, 'n', 'n', 2.f, 1.3f);
        prod(C2, A2, B2, 'n', 'n', 2.f, 1.3f);
        mat_eq(C, C2, "spmv_dev_correctness");
    }
    {   // host DIA vs dense (:130-143): C = 1.3*C + 2*A_dense*B computed densely in double
        sequence(B); sequence(C);
        tensor<float, host_memory_space, column_major> A_(n, m), Cd(n, k);
        convert(A_, A);
        for (int i = 0; i < n; i++)
            for (int c = 0; c < k; c++) {
                double s = 0;
                for (int j = 0; j < m; j++) s += (double)(float)A_(i, j) * (double)(float)B(j, c);
                Cd(i, c) = (float)(1.3f * (double)(float)C(i, c) + 2.0 * s);
            }
        tensor<float, dev_memory_space, column_major> C2(C.shape()), B2(B.shape());
        convert(C2, C); convert(B2, B);
        prod(C2, A2, B2, 'n', 'n', 2.f, 1.3f);
        mat_cmp(C2, Cd, 0.1, "spmv dev DIA vs dense");
    }
    {   // spmv on packed vectors
        tensor<float, host_memory_space> v(m * 2), d(n * 2);
        sequence(v); fill(d, 0);
        tensor<float, dev_memory_space> v2(m * 2), d2(n * 2);
        v2 = v; d2 = d;
        spmv(d, A, v, 'n', 1.f, 0.f);
        spmv(d2, A2, v2, 'n', 1.f, 0.f);
        int bad = 0;
        for (int i = 0; i < n * 2; i++) bad += (float)d[i] != (float)d2[i];
        CHECK(bad == 0);
    }
    {   // preconditions throw, as cuvAssert does
        tensor<float, dev_memory_space, column_major> C2(C.shape()), B2(B.shape());
        bool threw = false;
        try { prod(C2, A2, B2, 'n', 't'); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
        threw = false;
        try { prod(B2, A2, C2, 'n', 'n'); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);
    }
}

// ---- densedense_to_dia.cpp -----------------------------------------------------------------------------
static void test_dd2dia() {
    const int n = 36, m = 19, k = 16, rf = 4;
    dia_matrix<float, dev_memory_space> C(n, m, 7, std::max(n, m), rf);
    tensor<float, dev_memory_space, column_major> A(n, k), B(m, k);
    std::vector<int> off;
    for (int i = -C.num_dia() / 2; i <= C.num_dia() / 2; i++) off.push_back(i);
    C.set_offsets(off);
    fill(C.vec(), 0); sequence(A); sequence(B);
    dia_matrix<float, host_memory_space> C2(n, m, C.num_dia(), C.stride(), rf);
    tensor<float, host_memory_space, column_major> A2(A.shape()), B2(B.shape());
    convert(C2, C); convert(A2, A); convert(B2, B);
    dev_block_descriptor<float> bd(C);
    host_block_descriptor<float> bdh(C2);
    densedense_to_dia(C, bd, A, B);
    densedense_to_dia(C2, bdh, A2, B2);
    {   // dd2s_cmp_dev_host (:166-197)
        int bad = 0;
        for (int i = 0; i < n; i++)
            for (int j = 0; j < m; j++) bad += (float)C(i, j) != (float)C2(i, j);
        CHECK(bad == 0);
    }
    {   // dd2s_correctness_dev (:109-137): stored cells equal the dense A*B^T
        int bad = 0, stored = 0;
        for (int i = 0; i < n; i++)
            for (int j = 0; j < m; j++) {
                if (!C.has(i, j)) { bad += C(i, j) != 0.f; continue; }
                double s = 0;
                for (int b = 0; b < k; b++) s += (double)(float)A2(i, b) * (double)(float)B2(j, b);
                stored++;
                bad += std::fabs((float)C(i, j) - s) > 1e-4 * std::fabs(s);
            }
        CHECK(bad == 0);
        CHECK(stored > 100);
    }
    {   // non-default factors: C = 0.5*C + 0.25*A*B^T, device vs host
        densedense_to_dia(C, bd, A, B, 0.25f, 0.5f);
        densedense_to_dia(C2, bdh, A2, B2, 0.25f, 0.5f);
        int bad = 0;
        for (int i = 0; i < n; i++)
            for (int j = 0; j < m; j++) {
                const float a = C(i, j), b = C2(i, j);
                bad += std::fabs(a - b) > 1e-5f * std::fabs(b);
            }
        CHECK(bad == 0);
    }
}

// ---- dia_mat.cpp / convert.cpp ----------------------------------------------------------------------------
static void test_dia_mat() {
    const int n = 32, m = 16;
    dia_matrix<float, host_memory_space> w(n, m, 3, n);
    std::vector<int> off = {0, 1, -1};
    w.set_offsets(off);
    sequence(w.vec());
    {   // spmv_uninit (:103-108): converting into an empty device matrix allocates it
        dia_matrix<float, dev_memory_space> w2;
        convert(w2, w);
        CHECK(w2.vec_ptr() != nullptr && w2.h() == (unsigned)n && w2.w() == (unsigned)m && w2.num_dia() == 3);
    }
    {   // save / load (:84-101): the seven serialised fields survive a round trip, as does the device copy
        const std::string fn = "/tmp/cuvdia_test_matrix.bin";
        save_dia_matrix(w, fn);
        dia_matrix<float, host_memory_space> w2;
        load_dia_matrix(w2, fn);
        std::remove(fn.c_str());
        CHECK(w2.h() == w.h() && w2.w() == w.w() && w2.num_dia() == w.num_dia() && w2.stride() == w.stride() &&
              w2.row_fact() == w.row_fact());
        int bad = 0;
        for (int i = 0; i < n; i++) for (int j = 0; j < m; j++) bad += (float)w(i, j) != (float)w2(i, j);
        for (int s = 0; s < 3; s++) bad += w2.get_offset(s) != off[s];
        CHECK(bad == 0);
    }
    {   // dia2dense (:111-119)
        tensor<float, host_memory_space, column_major> w2(n, m);
        convert(w2, w);
        int bad = 0;
        for (int i = 0; i < n; i++) for (int j = 0; j < m; j++) bad += (float)w2(i, j) != (float)w(i, j);
        CHECK(bad == 0);
    }
    {   // host2dev and back (:121-132, convert.cpp:110-129)
        dia_matrix<float, dev_memory_space> w2(n, m, w.num_dia(), w.stride());
        convert(w2, w);
        dia_matrix<float, host_memory_space> w3(n, m, w.num_dia(), w.stride());
        convert(w3, w2);
        int bad = 0;
        for (int i = 0; i < n; i++) for (int j = 0; j < m; j++) bad += (float)w(i, j) != (float)w3(i, j) || (float)w(i, j) != (float)w2(i, j);
        CHECK(bad == 0);
        for (int s = 0; s < 3; s++) CHECK(w3.get_offset(s) == off[s] && w2.get_offset(s) == off[s]);
        // avg_diagonals (:134-142; the call is commented out in CUV's test): device == host definition
        tensor<float, host_memory_space> avg_h(w.num_dia());
        tensor<float, dev_memory_space> avg_d(w.num_dia());
        avg_diagonals(avg_h, w);
        avg_diagonals(avg_d, w2);
        for (int s = 0; s < 3; s++) CHECK(std::fabs((float)avg_h[s] - (float)avg_d[s]) <= 1e-5f * std::fabs((float)avg_h[s]) + 1e-7f);
    }
}

// ---- matrix_op.cpp reductions -----------------------------------------------------------------------------
template <class L> static void reduce_sweep(const char* layout) {
    const int n = 270;
    tensor<float, host_memory_space, L> h(n, n);
    unsigned s = 12345;
    for (int i = 0; i < n * n; i++) { s = s * 1664525u + 1013904223u; h[i] = (float)((s >> 8) & 0xffff) / 65536.f + 0.5f; }
    tensor<float, dev_memory_space, L> d(n, n);
    convert(d, h);
    const reduce_functor rfs[] = {RF_ADD, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX, RF_ARGMIN, RF_MIN, RF_MULT, RF_LOGADDEXP, RF_ADDEXP};
    for (reduce_functor rf : rfs)
        for (int to_col = 0; to_col < 2; to_col++) {
            tensor<float, host_memory_space> vh(n);
            tensor<float, dev_memory_space> vd(n);
            fill(vh, 0); fill(vd, 0);
            if (to_col) { reduce_to_col(vh, h, rf); reduce_to_col(vd, d, rf); }
            else { reduce_to_row(vh, h, rf); reduce_to_row(vd, d, rf); }
            int bad = 0;
            for (int i = 0; i < n; i++) {
                const float a = vh[i], b = vd[i];
                const bool exact = rf == RF_MAX || rf == RF_MIN || rf == RF_ARGMAX || rf == RF_ARGMIN;
                bad += exact ? (a != b) : !(std::fabs(a - b) <= 1e-3f * std::fabs(a));      // CUV: 0.1 %
            }
            if (bad) std::printf("reduce %s rf=%d to_col=%d: %d mismatches\n", layout, (int)rf, to_col, bad);
            CHECK(bad == 0);
        }
    {   // factors (matrix_op.cpp:721-737 pattern): v = 0.5*v + 1.0*sum
        tensor<float, host_memory_space> vh(n);
        tensor<float, dev_memory_space> vd(n);
        sequence(vh); sequence(vd);
        reduce_to_col(vh, h, RF_ADD, 1.f, 0.5f);
        reduce_to_col(vd, d, RF_ADD, 1.f, 0.5f);
        int bad = 0;
        for (int i = 0; i < n; i++) bad += !(std::fabs((float)vh[i] - (float)vd[i]) <= 1e-4f * std::fabs((float)vh[i]));
        CHECK(bad == 0);
    }
}

// reduce_to_col / reduce_to_row between the other element types CUV instantiates (matrix_ops_reduce.cu:395-413;
// CUV's own test of a typed pair: src/tests/matrix_op.cpp:574-628 compares device with host): device == host, exactly.
template <class V, class V2> static void reduce_typed_pair(const char* what, int modulus) {
    const int n = 200, m = 60;
    tensor<V, host_memory_space, column_major> h(n, m);
    unsigned s = 777;
    for (int i = 0; i < n * m; i++) { s = s * 1664525u + 1013904223u; h[i] = (V)(((s >> 10) % modulus)); }
    tensor<V, dev_memory_space, column_major> d(n, m);
    convert(d, h);
    const reduce_functor rfs[] = {RF_ADD, RF_MAX, RF_MIN, RF_ARGMAX, RF_ARGMIN};
    for (reduce_functor rf : rfs)
        for (int to_col = 0; to_col < 2; to_col++) {
            const int len = to_col ? n : m;
            tensor<V2, host_memory_space> vh(len);
            tensor<V2, dev_memory_space> vd(len);
            if (to_col) { reduce_to_col(vh, h, rf); reduce_to_col(vd, d, rf); }
            else { reduce_to_row(vh, h, rf); reduce_to_row(vd, d, rf); }
            tensor<V2, host_memory_space> back(len);
            back = vd;
            int bad = 0;
            for (int i = 0; i < len; i++) bad += !((V2)vh[i] == (V2)back[i]);
            if (bad) std::printf("typed reduce %s rf=%d to_col=%d: %d mismatches\n", what, (int)rf, to_col, bad);
            CHECK(bad == 0);
        }
}
static void test_reduce_typed() {
    reduce_typed_pair<int, float>("int -> float", 1000);
    reduce_typed_pair<unsigned int, float>("unsigned -> float", 1000);
    reduce_typed_pair<unsigned char, float>("uchar -> float", 2);          // line totals stay inside 8 bits
    reduce_typed_pair<float, int>("float -> int", 100);
    reduce_typed_pair<float, unsigned int>("float -> unsigned", 100);
    reduce_typed_pair<float, unsigned char>("float -> uchar", 2);
    reduce_typed_pair<unsigned char, unsigned char>("uchar -> uchar", 2);
    reduce_typed_pair<unsigned char, unsigned int>("uchar -> unsigned", 2);
}

// filter_factory (basics/filter_factory.hpp:43-76): the diagonals of a convolution layer, and a filter read back.
static void test_filter_factory() {
    filter_factory<float, host_memory_space> ff(12, 12, 3, 1, 1);
    dia_matrix<float, host_memory_space>* m = ff.get_dia();
    CHECK(m->h() == 144 && m->w() == 144 && m->num_dia() == 9 && m->stride() == 144);
    CHECK(m->get_offset(0) == -13 && m->get_offset(4) == 0 && m->get_offset(8) == 13);
    fill(m->vec(), 0.f);
    const std::vector<int> off = ff.offsets();
    for (int t = 0; t < 9; t++) m->set(100 - off[t], 100, (float)(t + 1));
    tensor<float, host_memory_space, row_major>* f = ff.extract_filter(*m, 100);
    bool ok = f->size() == 9;
    for (int t = 0; t < 9 && ok; t++) ok = (float)(*f)[t] == (float)(9 - t);
    CHECK(ok);
    delete f;
    delete m;
    filter_factory<float, dev_memory_space> fd(16, 16, 5, 2, 3);
    dia_matrix<float, dev_memory_space>* md = fd.get_dia();
    CHECK(md->num_dia() == 100 && md->h() == 512 && md->w() == 768);
    delete md;
}

static void test_tensor_ops() {
    tensor<float, host_memory_space> a(100), b(100);
    sequence(a); fill(b, 2.f);
    tensor<float, dev_memory_space> a2(100), b2(100);
    a2 = a; b2 = b;
    apply_binary_functor(a, b, BF_AXPBY, 0.9f, -0.01f);
    apply_binary_functor(a2, b2, BF_AXPBY, 0.9f, -0.01f);
    int bad = 0;
    for (int i = 0; i < 100; i++) bad += (float)a[i] != (float)a2[i];
    CHECK(bad == 0);
    apply_binary_functor(a, b, BF_MULT); apply_binary_functor(a2, b2, BF_MULT);
    apply_binary_functor(a, a, b, BF_SUBTRACT); apply_binary_functor(a2, a2, b2, BF_SUBTRACT);
    for (int i = 0; i < 100; i++) bad += (float)a[i] != (float)a2[i];
    CHECK(bad == 0);
    tensor<float, dev_memory_space> alias = a2;          // same-type assignment aliases the storage
    CHECK(alias.ptr() == a2.ptr());
}

// ---- optimize.cpp: the gradient step minimises f(W) = 2 (W - optimum)^2 -------------------------------------
template <class M> static void lswd_optimization(int N, bool momentum, const char* what) {
    tensor<float, host_memory_space> h_opt(N), h_w(N);
    unsigned s = 12345u;
    for (int i = 0; i < N; i++) { s = s * 1664525u + 1013904223u; h_opt[i] = (s >> 8) * (1.f / 16777216.f); }
    for (int i = 0; i < N; i++) { s = s * 1664525u + 1013904223u; h_w[i] = (s >> 8) * (1.f / 16777216.f); }
    tensor<float, M> W(N), dW(N), mom(N), optimum(N);
    W = h_w; optimum = h_opt;
    fill(mom, 0.f);
    const int max_iter = 1000;
    for (int iter = 0; iter < max_iter; ++iter) {
        apply_binary_functor(dW, W, optimum, BF_SUBTRACT);
        if (momentum) learn_step_weight_decay_momentum(W, mom, dW, 0.01f, 1.f - iter / (float)max_iter, 0.0f);
        else learn_step_weight_decay(W, dW, 0.01f, 0.0f);
    }
    tensor<float, host_memory_space> res(N);
    res = W;
    int bad = 0;
    double err = 0;
    for (int i = 0; i < N; i++) {
        const float a = (float)res[i] + 1.f, b = (float)h_opt[i] + 1.f;
        bad += !(std::fabs(a - b) <= 1e-4f * std::max(std::fabs(a), std::fabs(b)));     // BOOST_CHECK_CLOSE 0.01 %
        err += 2.0 * ((float)res[i] - (float)h_opt[i]) * ((float)res[i] - (float)h_opt[i]);
    }
    g_checks++;
    if (bad || !(err / N <= 1e-4)) { g_fail++; std::printf("FAILED %s: %d weights off the optimum, mean error %g\n", what, bad, err / N); }
}

static void test_learn_step() {
    lswd_optimization<host_memory_space>(8092, false, "lswd host");
    lswd_optimization<dev_memory_space>(8092, false, "lswd dev");
    lswd_optimization<host_memory_space>(8092, true, "lswd momentum host");
    lswd_optimization<dev_memory_space>(8092, true, "lswd momentum dev");
    // host and device objects of the same template agree bit for bit, decay included, on a DIA matrix's values
    const int n = 96, nd = 5;
    dia_matrix<float, host_memory_space> Wh(n, n, nd, n), Gh(n, n, nd, n);
    std::vector<int> off = {-2, -1, 0, 1, 2};
    Wh.set_offsets(off); Gh.set_offsets(off);
    sequence(Wh.vec()); sequence(Gh.vec());
    apply_binary_functor(Gh.vec(), Wh.vec(), BF_AXPBY, 0.37f, -0.001f);
    dia_matrix<float, dev_memory_space> Wd(n, n, nd, n), Gd(n, n, nd, n);
    convert(Wd, Wh); convert(Gd, Gh);
    learn_step_weight_decay(Wh, Gh, 0.03f, 0.2f);
    learn_step_weight_decay(Wd, Gd, 0.03f, 0.2f);
    dia_matrix<float, host_memory_space> back(n, n, nd, n);
    convert(back, Wd);
    int bad = 0;
    for (unsigned i = 0; i < Wh.vec().size(); i++) bad += (float)Wh.vec()[i] != (float)back.vec()[i];
    CHECK(bad == 0);
}

// ---- matrix_op.cpp:574-628: reductions of a 3-D tensor (the leading or the trailing dimension survives) --------
static void test_reduce_3d() {
    tensor<float, dev_memory_space> Md(extents[5][4][3]);
    tensor<float, host_memory_space> Mh(extents[5][4][3]);
    sequence(Md); sequence(Mh);
    {
        tensor<float, dev_memory_space> vd(extents[3]);
        tensor<float, host_memory_space> vh(extents[3]);
        sequence(vd); sequence(vh);
        reduce_to_row(vd, Md);
        reduce_to_row(vh, Mh);
        for (int k = 0; k < 3; k++) {
            float sum = 0.f;
            for (int i = 0; i < 5; i++)
                for (int j = 0; j < 4; j++) sum += (float)Mh(i, j, k);
            CHECK(std::fabs((float)vd[k] - (float)vh[k]) <= 1e-4f * std::fabs((float)vh[k]));
            CHECK(std::fabs((float)vh[k] - sum) <= 1e-4f * std::fabs(sum));
        }
    }
    {
        tensor<float, dev_memory_space> vd(extents[5]);
        tensor<float, host_memory_space> vh(extents[5]);
        sequence(vd); sequence(vh);
        reduce_to_col(vd, Md);
        reduce_to_col(vh, Mh);
        for (int i = 0; i < 5; i++) {
            float sum = 0.f;
            for (int j = 0; j < 4; j++)
                for (int k = 0; k < 3; k++) sum += (float)Mh(i, j, k);
            CHECK(std::fabs((float)vd[i] - (float)vh[i]) <= 1e-4f * std::fabs((float)vh[i]));
            CHECK(std::fabs((float)vh[i] - sum) <= 1e-4f * std::fabs(sum));
        }
    }
}

// A kernel that gave up a bounded wait must surface as an exception from the next blocking call, as a failed
// operation does in CUV (tools/cuv_general.cu:51-61); the self-test kernel leaves the code without any fault.
static void test_given_up_wait_throws() {
    const int n = 64, k = 8;
    dia_matrix<float, dev_memory_space> A(n, n, 3, n);
    std::vector<int> off = {-1, 0, 1};
    A.set_offsets(off);
    fill(A.vec(), 1.f);
    tensor<float, dev_memory_space, column_major> B(n, k), C(n, k);
    fill(B, 1.f);
    prod(C, A, B);                                   // healthy call
    CHECK((float)C(5, 0) == 3.f);
    cuvdia_check(cuvdia_selftest_bounded_wait(A.plan(), 1000, 0));
    bool thrown = false;
    try { prod(C, A, B); } catch (const std::runtime_error& e) {
        thrown = std::string(e.what()).find("gave up a bounded wait") != std::string::npos;
    }
    CHECK(thrown);
    prod(C, A, B);                                   // the word was cleared: the next call is clean again
    CHECK((float)C(5, 0) == 3.f);
    cuvdia_check(cuvdia_selftest_bounded_wait(A.plan(), 1000, 0));
    dev_block_descriptor<float> bd(A);
    thrown = false;
    try { densedense_to_dia(A, bd, C, B); } catch (const std::runtime_error&) { thrown = true; }
    CHECK(thrown);
}

// fill_rnd_uniform and rnd_binarize (random/random.hpp:48-55): the device numbers are the host restatement's, a second
// call draws other numbers, re-seeding starts over, and a binarised tensor is the comparison with those numbers.
static void test_random() {
    const int h = 37, w = 21;                        // 37 rows: the last group of four is ragged
    tensor<float, dev_memory_space, column_major> U(h, w), U2(h, w);
    initialize_mersenne_twister_seeds(99);
    fill_rnd_uniform(U);
    fill_rnd_uniform(U2);
    std::vector<float> r0((size_t)h * w), r1((size_t)h * w);
    oracle_uniform(r0.data(), h, h, w, 99, 0, 0, 0);
    oracle_uniform(r1.data(), h, h, w, 99, 1, 0, 0);
    int bad = 0, same = 0;
    for (int j = 0; j < w; j++)
        for (int i = 0; i < h; i++) {
            const float a = U(i, j), b = U2(i, j);
            bad += a != r0[(size_t)j * h + i] || b != r1[(size_t)j * h + i] || !(a >= 0.f && a < 1.f);
            same += a == b;
        }
    CHECK(bad == 0);
    CHECK(same < h * w / 100);
    initialize_mersenne_twister_seeds(99);
    tensor<float, dev_memory_space, column_major> P(h, w);
    tensor<float, host_memory_space, column_major> Ph(h, w);
    for (int j = 0; j < w; j++)
        for (int i = 0; i < h; i++) Ph(i, j) = (float)((i * 7 + j * 13) % 11) / 10.f;     // 0 .. 1 in tenths
    P = Ph;
    rnd_binarize(P);                                  // draw 0 after the re-seed: compares with r0
    bad = 0;
    int ones = 0;
    for (int j = 0; j < w; j++)
        for (int i = 0; i < h; i++) {
            const float want = (float)Ph(i, j) > r0[(size_t)j * h + i] ? 1.f : 0.f;
            bad += (float)P(i, j) != want;
            ones += want == 1.f;
        }
    CHECK(bad == 0);
    CHECK(ones > h * w / 4 && ones < 3 * h * w / 4);
    // a row-major tensor is drawn in memory order: its last dimension is the generator's row
    tensor<float, dev_memory_space, row_major> R(w, h);
    initialize_mersenne_twister_seeds(99);
    fill_rnd_uniform(R);
    bad = 0;
    for (int j = 0; j < w; j++)
        for (int i = 0; i < h; i++) bad += (float)R(j, i) != r0[(size_t)j * h + i];
    CHECK(bad == 0);
    tensor<float, dev_memory_space, column_major> v1(50);
    initialize_mersenne_twister_seeds(3);
    fill_rnd_uniform(v1);
    std::vector<float> rv(50);
    oracle_uniform(rv.data(), 50, 50, 1, 3, 0, 0, 0);
    bad = 0;
    for (int i = 0; i < 50; i++) bad += (float)v1(i) != rv[i];
    CHECK(bad == 0);
}

int main() {
    try {
        initCUDA(0);
        test_spmv();
        test_dd2dia();
        test_dia_mat();
        reduce_sweep<column_major>("column_major");
        reduce_sweep<row_major>("row_major");
        test_tensor_ops();
        test_filter_factory();
        test_reduce_typed();
        test_reduce_3d();
        test_learn_step();
        test_random();
        test_given_up_wait_throws();
        exitCUDA();
    } catch (const std::exception& e) {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%d checks, %d failed, %llu kernels launched through libcuvdia\n", g_checks, g_fail, cuvdia_launch_count());
    return g_fail ? 1 : 0;
}
