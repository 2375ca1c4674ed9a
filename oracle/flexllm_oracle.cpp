// CPU oracle for the quantized Llama-3.2-1B operator path of FlexLLM.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is a plain array-based C++ restatement of the
// reference's HLS operator templates (FlexLLM `Modules/*.h`), written to be the checker
// that the CUDA kernels are compared against. Nothing in the product library links,
// loads or calls it.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fno-fast-math -fopenmp (x86-64 baseline
// ISA, so no fused multiply-add is ever generated: every fp32 operation is rounded on
// its own, as in a default C-simulation build of the reference).
//
// Parity status: pinned. Every function below is checked bit-for-bit against the
// reference's own templates, compiled unmodified through the header shim in
// oracle/ref_shim (see oracle/ref_wrap.cpp), and against fixtures generated from them.
//
// Conventions: all tensors row-major, weights [N][K] with K contiguous. `rnd` is
// std::round (half away from zero). (float)int32 is round-to-nearest-even.

#include <omp.h>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

#define ORC_API extern "C" __attribute__((visibility("default")))

// exp() flavour. The reference calls `exp(float)` = the C library's expf, whose last-bit rounding is
// implementation-defined (glibc's differs from the correctly rounded value on about 0.06 % of
// inputs). Mode 0: the libm expf of the build machine (what a C-simulation of the reference computes
// here). Mode 1: the correctly rounded single-precision exponential, (float)exp((double)x), which
// the CUDA kernels reproduce bit for bit.
static int g_exp_mode = 0;
ORC_API void orc_set_exp_mode(int mode) { g_exp_mode = mode; }
// Threads of the OpenMP loops below (a launcher may have exported OMP_NUM_THREADS=1 before this library was loaded).
ORC_API void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
ORC_API int orc_get_threads(void) { return omp_get_max_threads(); }
ORC_API int orc_get_exp_mode() { return g_exp_mode; }

namespace {

inline float ref_exp(float x) { return g_exp_mode ? (float)std::exp((double)x) : std::exp(x); }

inline float absf(float x) { return std::fabs(x); }

// Symmetric scale from running max/min (quant.h:84-96): max starts at -1e32, min at 1e32.
inline float sym_scale(const float* x, long n, float scale_base) {
    float mx = -1e32f, mn = 1e32f;
    for (long k = 0; k < n; k++) {
        if (x[k] > mx) mx = x[k];
        if (x[k] < mn) mn = x[k];
    }
    float a = absf(mx), b = absf(mn);
    float s = (a > b ? a : b) / scale_base;
    if (s == 0) s = 1;
    return s;
}

// In-place Walsh-Hadamard butterflies in the stride order that reproduces the reference's
// Omega network (FHT.h:31-53) bit for bit: h = 2, 4, ..., N/2, then 1.
inline void fht_inplace(float* z, int N) {
    auto stage = [&](int h) {
        for (int i = 0; i < N; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = z[j], b = z[j + h];
                z[j] = a + b;
                z[j + h] = a - b;
            }
    };
    for (int h = 2; h < N; h <<= 1) stage(h);
    stage(1);
}

// Softmax over x[0..len) following Softmax.h:25-161 (prefill) / :474-634 (decode):
// running max from -1e32, four partial sums over k mod 4 in increasing k, combined
// (p0+p1)+(p2+p3), r = 1/total, P = e*r.  `e` may alias x.
inline void softmax_row(const float* x, int len, float* p) {
    float mx = -1e32f;
    for (int k = 0; k < len; k++) mx = x[k] > mx ? x[k] : mx;
    float ps[4] = {0, 0, 0, 0};
    for (int k = 0; k < len; k++) {
        float e = ref_exp(x[k] - mx);
        p[k] = e;
        ps[k & 3] += e;
    }
    float r = 1.0f / ((ps[0] + ps[1]) + (ps[2] + ps[3]));
    for (int k = 0; k < len; k++) p[k] = p[k] * r;
}

inline float silu(float g) { return g / (1 + ref_exp(-g)); }  // Swish.h:19

} // namespace

// ----------------------------------------------------------------------------------------------
// A.1  dynamic per-token symmetric quantisation, 8 bit  (quant.h:6-112 sym branch; :332-431)
// ----------------------------------------------------------------------------------------------
ORC_API void orc_quant_per_token(const float* x, int M, int K, int8_t* q, float* s) {
#pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const float* xr = x + (long)m * K;
        float sc = sym_scale(xr, K, 127.0f);
        s[m] = sc;
        for (int k = 0; k < K; k++) q[(long)m * K + k] = (int8_t)(long long)std::round(xr[k] / sc);
    }
}

// Asymmetric per-token quantiser, `bits` bits (the reference's shipped configuration: 4-bit asymmetric activations in
// front of every linear layer; quant.h:53-81): s = (max - min) / (2^bits - 1) (0 -> 1), zero point b = min,
// q = (unsigned) round((x - b) / s), in [0, 2^bits - 1] by construction.
ORC_API void orc_quant_per_token_asym(const float* x, int M, int K, int bits, uint8_t* q, float* s, float* b) {
    const float base = (float)((1 << bits) - 1);
    const long long mask = (1ll << bits) - 1;
#pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const float* xr = x + (long)m * K;
        float mx = -1e32f, mn = 1e32f;
        for (int k = 0; k < K; k++) { if (xr[k] > mx) mx = xr[k]; if (xr[k] < mn) mn = xr[k]; }
        float sc = (mx - mn) / base;
        if (sc == 0) sc = 1;
        s[m] = sc; b[m] = mn;
        for (int k = 0; k < K; k++) {
            const float t = (xr[k] - mn) / sc;
            q[(long)m * K + k] = (uint8_t)((long long)std::round(t) & mask);
        }
    }
}

// Dequant with the zero point (quant.h:146-148): y = ((float)acc * s_tok) * s_ch + b_tok * wsum, where
// wsum[n] = sum_k w[n][k] * s_ch[n] comes with the checkpoint (Linear_Layer_Prefilling_tb.cpp:222-237).
ORC_API void orc_dequant_asym(const int32_t* acc, const float* s_tok, const float* b_tok, const float* s_ch, const float* wsum, int M,
                              int N, float* y) {
#pragma omp parallel for
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float t = (float)acc[(long)m * N + n] * s_tok[m];
            t = t * s_ch[n];
            const float z = b_tok[m] * wsum[n];
            y[(long)m * N + n] = t + z;
        }
}

// ----------------------------------------------------------------------------------------------
// A.2  exact integer matmul  acc[m][n] = sum_k a[m][k]*w[n][k]   (PE.h:526-583, MHA.h:113-187)
// ----------------------------------------------------------------------------------------------
__attribute__((target_clones("avx2", "default")))
static void gemm_s8_rows(const int8_t* a, const int8_t* w, int N, int K, int32_t* acc) {
    for (int n = 0; n < N; n++) {
        const int8_t* wr = w + (long)n * K;
        int32_t t = 0;
        for (int k = 0; k < K; k++) t += (int32_t)a[k] * (int32_t)wr[k];
        acc[n] = t;
    }
}
__attribute__((target_clones("avx2", "default")))
static void gemm_u8_rows(const uint8_t* a, const int8_t* w, int N, int K, int32_t* acc) {
    for (int n = 0; n < N; n++) {
        const int8_t* wr = w + (long)n * K;
        int32_t t = 0;
        for (int k = 0; k < K; k++) t += (int32_t)a[k] * (int32_t)wr[k];
        acc[n] = t;
    }
}

ORC_API void orc_gemm_s8s8(const int8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
#pragma omp parallel for
    for (int m = 0; m < M; m++) gemm_s8_rows(a + (long)m * K, w, N, K, acc + (long)m * N);
}
ORC_API void orc_gemm_u8s8(const uint8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
#pragma omp parallel for
    for (int m = 0; m < M; m++) gemm_u8_rows(a + (long)m * K, w, N, K, acc + (long)m * N);
}

// ----------------------------------------------------------------------------------------------
// A.3  dequant  y = ((float)acc * s_tok[m]) * s_ch[n]     (quant.h:151; decode :461, :513)
// ----------------------------------------------------------------------------------------------
ORC_API void orc_dequant(const int32_t* acc, const float* s_tok, const float* s_ch, int M, int N, float* y) {
#pragma omp parallel for
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float t = (float)acc[(long)m * N + n] * s_tok[m];
            y[(long)m * N + n] = t * s_ch[n];
        }
}

// ----------------------------------------------------------------------------------------------
// A.5  Walsh-Hadamard transform, natural order, divided by `scale`   (FHT.h:7-129)
// ----------------------------------------------------------------------------------------------
ORC_API void orc_fht(const float* x, long rows, int N, float scale, float* y) {
#pragma omp parallel for
    for (long r = 0; r < rows; r++) {
        std::vector<float> z(x + r * N, x + (r + 1) * N);
        fht_inplace(z.data(), N);
        for (int k = 0; k < N; k++) y[r * N + k] = z[k] / scale;
    }
}

// ----------------------------------------------------------------------------------------------
// A.4  half-split RoPE by table, head_dim 64    (RoPE.h:61-90, :143-171)
// x, y: [T][H][64]; pos: [T]; cos_t/sin_t: [P][32]
// ----------------------------------------------------------------------------------------------
ORC_API void orc_rope(const float* x, const int* pos, const float* cos_t, const float* sin_t,
                      long T, int H, float* y) {
#pragma omp parallel for
    for (long t = 0; t < T; t++) {
        const float* c = cos_t + (long)pos[t] * 32;
        const float* s = sin_t + (long)pos[t] * 32;
        for (int h = 0; h < H; h++) {
            const float* xi = x + (t * H + h) * 64;
            float* yo = y + (t * H + h) * 64;
            for (int k = 0; k < 32; k++) {
                float x0 = xi[k], x1 = xi[k + 32];
                float o0 = x0 * c[k] - x1 * s[k];
                float o1 = x0 * s[k] + x1 * c[k];
                yo[k] = o0;
                yo[k + 32] = o1;
            }
        }
    }
}

// llama3 RoPE table (formula in the comment at RoPE.h:28-51), evaluated in double and
// rounded to fp32. theta=500000, factor 32, low 1, high 4, original context 8192.
ORC_API void orc_rope_table(int P, float* cos_t, float* sin_t) {
    const double theta = 500000.0, factor = 32.0, lowf = 1.0, highf = 4.0, orig = 8192.0;
    const double PI = 3.14159265358979323846;
    for (int i = 0; i < 32; i++) {
        double inv = std::pow(theta, (2.0 * i) / 64.0);
        double f = 1.0 / inv;
        double wl = 2.0 * PI * inv;
        double sf;
        if (wl < orig / highf) sf = f;
        else if (wl > orig / lowf) sf = f / factor;
        else {
            double a = (orig / wl - lowf) / (highf - lowf);
            sf = (1 - a) * (f / factor) + a * f;
        }
        for (int p = 0; p < P; p++) {
            double th = p * sf;
            cos_t[(long)p * 32 + i] = (float)std::cos(th);
            sin_t[(long)p * 32 + i] = (float)std::sin(th);
        }
    }
}

// ----------------------------------------------------------------------------------------------
// A.6  softmax rows. valid[r] (may be NULL) = number of leading unmasked entries of row r;
// entries k >= valid[r] are replaced by -1e32 first (MHA.h:262-267).
// ----------------------------------------------------------------------------------------------
ORC_API void orc_softmax(const float* x, long rows, int len, const int* valid, float* p) {
#pragma omp parallel for
    for (long r = 0; r < rows; r++) {
        std::vector<float> t(x + r * len, x + (r + 1) * len);
        if (valid)
            for (int k = valid[r]; k < len; k++) t[k] = -1e32f;
        softmax_row(t.data(), len, p + r * len);
    }
}

// ----------------------------------------------------------------------------------------------
// A.8  RMSNorm. lanes == 0: prefill order (LayerNorm.h:82-130). lanes > 0: decode order with
// `lanes` contiguous chunks (LayerNorm.h:263-321).
// ----------------------------------------------------------------------------------------------
static float rms_recip(const float* x, int D, float eps, int lanes) {
    float tot;
    if (lanes == 0) {
        float ss[4] = {0, 0, 0, 0};
        for (int k = 0; k < D; k++) ss[k & 3] += x[k] * x[k];
        tot = (ss[0] + ss[1]) + (ss[2] + ss[3]);
    } else {
        int C = D / lanes;
        tot = 0;
        for (int i = 0; i < lanes; i++) {
            float ss[4] = {0, 0, 0, 0};
            for (int k = 0; k < C; k++) { float v = x[i * C + k]; ss[k & 3] += v * v; }
            tot += (ss[0] + ss[1]) + (ss[2] + ss[3]);
        }
    }
    return 1.0f / std::sqrt(tot / D + eps);
}

ORC_API void orc_rmsnorm(const float* x, const float* gamma, int M, int D, float eps, int lanes, float* y) {
#pragma omp parallel for
    for (int m = 0; m < M; m++) {
        const float* xr = x + (long)m * D;
        float r = rms_recip(xr, D, eps, lanes);
        for (int k = 0; k < D; k++) y[(long)m * D + k] = xr[k] * r * gamma[k];
    }
}

// ----------------------------------------------------------------------------------------------
// A.10  SiLU, gate, residual    (Swish.h:19,:37; Linear_Layer.h:612-630; Residual_Layer.h:46-87)
// ----------------------------------------------------------------------------------------------
ORC_API void orc_silu(const float* g, long n, float* y) {
#pragma omp parallel for
    for (long i = 0; i < n; i++) y[i] = silu(g[i]);
}
ORC_API void orc_silu_mul(const float* g, const float* u, long n, float* y) {
#pragma omp parallel for
    for (long i = 0; i < n; i++) y[i] = silu(g[i]) * u[i];
}
ORC_API void orc_residual(const float* a, const float* b, long n, float* y) {
#pragma omp parallel for
    for (long i = 0; i < n; i++) y[i] = a[i] + b[i];
}

// ----------------------------------------------------------------------------------------------
// A.7  static symmetric quantisation  q = clamp(rnd(x / (f*s)))    (quant.h:252-295)
// is_signed: clamp to [-128,127]; else only the upper clamp at 255 (stored as a byte).
// x: [rows][n], s: per-row scale (rows entries) or a single scale when s_stride == 0.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_static_quant(const float* x, long rows, int n, const float* s, int s_stride,
                              float f, int is_signed, uint8_t* q) {
    const int base = is_signed ? 128 : 256;
#pragma omp parallel for
    for (long r = 0; r < rows; r++) {
        float d = f * s[r * s_stride];
        for (int k = 0; k < n; k++) {
            float t = x[r * n + k] / d;
            int v = (int)std::round(t);
            if (is_signed) v = v > base - 1 ? base - 1 : v < -base ? -base : v;
            else v = v > base - 1 ? base - 1 : v;
            q[r * n + k] = (uint8_t)v;
        }
    }
}

// ----------------------------------------------------------------------------------------------
// Greedy token = rank 0 of sort_top_k (Logits.h:5-31): strict '>' so ties keep the lowest index.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_argmax(const float* logits, int B, long V, int32_t* idx) {
#pragma omp parallel for
    for (int b = 0; b < B; b++) {
        const float* l = logits + (long)b * V;
        long best = 0;
        for (long v = 1; v < V; v++)
            if (l[v] > l[best]) best = v;
        idx[b] = (int32_t)best;
    }
}

// ----------------------------------------------------------------------------------------------
// Top-k sampling (Logits.h:145-279, as instantiated by the decode graphs: inner_block_parallel 1,
// enable_sub_max). `lanes` lanes each own a contiguous V/lanes slice of the vocabulary and keep an
// insertion-sorted top-k of it (sort_top_k, Logits.h:5-31: strict '>', so equal values stay in
// arrival order); the lanes' lists are merged by inserting rank 0 of every lane, then rank 1, ...
// (:215-224); softmax over the k winners with two interleaved partial sums (:232-247); the token is
// the first k whose cumulative probability exceeds the uniform number `rnd`, else the last (:252-271).
// Outputs: sampled index per row; optionally the merged top-k indices / values / probabilities.
// ----------------------------------------------------------------------------------------------
static void orc_sort_top_k(int* ids, float* vals, int top_k, int v_idx, float v) {
    int pos = top_k;
    for (int k = 0; k < top_k; k++)
        if (v > vals[k] && pos == top_k) pos = k;
    for (int k = top_k - 1; k >= 0; k--) {
        if (k > pos) { ids[k] = ids[k - 1]; vals[k] = vals[k - 1]; }
        else if (k == pos) { ids[k] = v_idx; vals[k] = v; }
    }
}
ORC_API int orc_topk_sample(const float* logits, int B, long V, int lanes, int top_k, const float* rnd, int32_t* idx,
                            int32_t* top_idx, float* top_val, float* top_prob) {
    if (top_k < 1 || top_k > 16 || lanes < 1 || V % lanes || V / lanes < top_k) return -1;
    const long seg = V / lanes;
    for (int b = 0; b < B; b++) {
        const float* l = logits + (long)b * V;
        std::vector<int> lid((size_t)lanes * top_k, -1);
        std::vector<float> lval((size_t)lanes * top_k, -1e32f);
        for (int i = 0; i < lanes; i++)
            for (long t = 0; t < seg; t++) orc_sort_top_k(&lid[(size_t)i * top_k], &lval[(size_t)i * top_k], top_k, (int)(i * seg + t), l[i * seg + t]);
        int fid[16]; float fval[16], prob[16], cdf[16];
        for (int k = 0; k < top_k; k++) { fid[k] = -1; fval[k] = -1e32f; }
        for (int K = 0; K < top_k; K++)
            for (int i = 0; i < lanes; i++) orc_sort_top_k(fid, fval, top_k, lid[(size_t)i * top_k + K], lval[(size_t)i * top_k + K]);
        float part[2] = {0.0f, 0.0f};
        for (int k = 0; k < top_k; k++) { prob[k] = ref_exp(fval[k] - fval[0]); part[k % 2] += prob[k]; }
        const float sum = part[0] + part[1];
        for (int k = 0; k < top_k; k++) prob[k] /= sum;
        cdf[0] = prob[0];
        for (int k = 1; k < top_k; k++) cdf[k] = prob[k] + cdf[k - 1];
        int sel = top_k - 1;
        for (int k = 0; k < top_k; k++)
            if (rnd[b] < cdf[k] && sel == top_k - 1) sel = k;
        idx[b] = fid[sel];
        for (int k = 0; k < top_k; k++) {
            if (top_idx) top_idx[(long)b * top_k + k] = fid[k];
            if (top_val) top_val[(long)b * top_k + k] = fval[k];
            if (top_prob) top_prob[(long)b * top_k + k] = prob[k];
        }
    }
    return 0;
}

// Token choice of orc_model_generate: greedy (top_k 0, the default) or top-k sampling with uniform numbers
// rnd [n_new][B] (row = output column).
static int g_sample_lanes = 0, g_sample_k = 0, g_sample_step = 0;
static const float* g_sample_rnd = nullptr;
ORC_API void orc_set_sampling(int lanes, int top_k, const float* rnd) { g_sample_lanes = lanes; g_sample_k = top_k; g_sample_rnd = rnd; }

// ----------------------------------------------------------------------------------------------
// Config 1: one W8A8 linear layer on already-quantised activations.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_linear_i8(const int8_t* a, const float* s_tok, const int8_t* w, const float* s_ch,
                           int M, int N, int K, int32_t* acc, float* y) {
    std::vector<int32_t> tmp;
    if (!acc) { tmp.resize((size_t)M * N); acc = tmp.data(); }
    orc_gemm_s8s8(a, w, M, N, K, acc);
    if (y) orc_dequant(acc, s_tok, s_ch, M, N, y);
}

// ----------------------------------------------------------------------------------------------
// Config 2: MLP block  (order of SpinQuant_Prefilling.h:1010-1049 / decode graph :1050-1126)
//   RMSNorm -> quant -> gate,up -> dequant -> silu(gate)*up -> FHT-8192/sqrt(8192) -> quant
//   -> down -> dequant -> + h
// lanes: RMSNorm order (0 = prefill, 8 = decode). Optional outputs may be NULL.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_mlp_block(const float* h, const float* gamma,
                           const int8_t* wg, const float* sg, const int8_t* wu, const float* su,
                           const int8_t* wd, const float* sd,
                           int M, int D, int F, float eps, int lanes, float fht_scale,
                           float* out,
                           int8_t* xq_out, float* xs_out,      // quantised RMSNorm output [M,D],[M]
                           float* act_out,                    // silu(g)*u [M,F]
                           int8_t* hq_out, float* hs_out,      // quantised FHT output [M,F],[M]
                           int32_t* down_acc_out) {           // [M,D]
    std::vector<float> xn((size_t)M * D), xs(M);
    std::vector<int8_t> xq((size_t)M * D);
    orc_rmsnorm(h, gamma, M, D, eps, lanes, xn.data());
    orc_quant_per_token(xn.data(), M, D, xq.data(), xs.data());
    std::vector<int32_t> acc((size_t)M * F);
    std::vector<float> g((size_t)M * F), u((size_t)M * F);
    orc_gemm_s8s8(xq.data(), wg, M, F, D, acc.data());
    orc_dequant(acc.data(), xs.data(), sg, M, F, g.data());
    orc_gemm_s8s8(xq.data(), wu, M, F, D, acc.data());
    orc_dequant(acc.data(), xs.data(), su, M, F, u.data());
    orc_silu_mul(g.data(), u.data(), (long)M * F, g.data());
    if (act_out) std::memcpy(act_out, g.data(), sizeof(float) * (size_t)M * F);
    orc_fht(g.data(), M, F, fht_scale, u.data());
    std::vector<int8_t> hq((size_t)M * F);
    std::vector<float> hs(M);
    orc_quant_per_token(u.data(), M, F, hq.data(), hs.data());
    std::vector<int32_t> dacc((size_t)M * D);
    std::vector<float> dn((size_t)M * D);
    orc_gemm_s8s8(hq.data(), wd, M, D, F, dacc.data());
    orc_dequant(dacc.data(), hs.data(), sd, M, D, dn.data());
    orc_residual(h, dn.data(), (long)M * D, out);
    if (xq_out) std::memcpy(xq_out, xq.data(), xq.size());
    if (xs_out) std::memcpy(xs_out, xs.data(), sizeof(float) * M);
    if (hq_out) std::memcpy(hq_out, hq.data(), hq.size());
    if (hs_out) std::memcpy(hs_out, hs.data(), sizeof(float) * M);
    if (down_acc_out) std::memcpy(down_acc_out, dacc.data(), sizeof(int32_t) * dacc.size());
}

// ----------------------------------------------------------------------------------------------
// Q/K preparation shared by configs 3 and 4:
//   x = (float)q_int * s  ->  RoPE(pos)  ->  FHT-64 / 8  ->  dynamic per-head-per-token int8
// (quant.h:242 dequant form; RoPE.h:61-90; FHT.h at N=64; quant.h:527-650 per-head quant).
// in: [T][H][64] int8 with scale [T][H];  out the same shapes.  do_rope = 0 skips the rotation.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_qk_prepare(const int8_t* q, const float* s, const int* pos,
                            const float* cos_t, const float* sin_t, long T, int H,
                            int8_t* q_out, float* s_out, float* rot_out) {
#pragma omp parallel for
    for (long t = 0; t < T; t++) {
        const float* c = cos_t + (long)pos[t] * 32;
        const float* sn = sin_t + (long)pos[t] * 32;
        for (int h = 0; h < H; h++) {
            long o = (t * H + h) * 64;
            float x[64], y[64];
            for (int k = 0; k < 64; k++) x[k] = (float)q[o + k] * s[t * H + h];
            for (int k = 0; k < 32; k++) {
                float x0 = x[k], x1 = x[k + 32];
                y[k] = x0 * c[k] - x1 * sn[k];
                y[k + 32] = x0 * sn[k] + x1 * c[k];
            }
            fht_inplace(y, 64);
            for (int k = 0; k < 64; k++) y[k] = y[k] / 8.0f;
            if (rot_out) std::memcpy(rot_out + o, y, sizeof(y));
            float sc = sym_scale(y, 64, 127.0f);
            s_out[t * H + h] = sc;
            for (int k = 0; k < 64; k++) q_out[o + k] = (int8_t)(long long)std::round(y[k] / sc);
        }
    }
}

// One attention row: scores for keys 0..nk-1 of one query head against one KV head.
//   acc   = sum_d q[d]*k[j][d]                       (MHA.h:189-243 / :615-669, exact)
//   score = (((float)acc * qs) * ks[j]) * 0.125f      (quant.h:242; 1/sqrt(64) folded, exact)
//   P     = softmax(score)                            (Softmax.h)
//   Pq    = min(rnd((P * vs[j]) / a_s), 255)  u8      (quant.h:262,279-280 unsigned static quant)
//   oacc  = sum_j Pq[j] * v[j][d]                     (MHA.h:339-389 / :854-907, exact u8 x s8)
//   out   = (float)oacc * a_s
// kp/vp/ksp/vsp give, for key j, pointers to its 64 bytes and its scale.
template <class KeyAt>
static void attn_row(const int8_t* q, float qs, int nk, KeyAt at, float a_s, float* out,
                     int32_t* oacc_out, uint8_t* p_out, float* score_out) {
    std::vector<float> sc(nk);
    for (int j = 0; j < nk; j++) {
        const int8_t* k; float ks; const int8_t* v; float vs;
        at(j, k, ks, v, vs);
        int32_t acc = 0;
        for (int d = 0; d < 64; d++) acc += (int32_t)q[d] * (int32_t)k[d];
        float t = (float)acc * qs;
        t = t * ks;
        sc[j] = t * 0.125f;
    }
    if (score_out) std::memcpy(score_out, sc.data(), sizeof(float) * nk);
    softmax_row(sc.data(), nk, sc.data());
    int32_t oacc[64] = {0};
    for (int j = 0; j < nk; j++) {
        const int8_t* k; float ks; const int8_t* v; float vs;
        at(j, k, ks, v, vs);
        float pt = sc[j] * vs;
        float t = pt / a_s;
        int r = (int)std::round(t);
        r = r > 255 ? 255 : r;
        uint8_t pq = (uint8_t)r;
        if (p_out) p_out[j] = pq;
        for (int d = 0; d < 64; d++) oacc[d] += (int32_t)pq * (int32_t)v[d];
    }
    for (int d = 0; d < 64; d++) {
        out[d] = (float)oacc[d] * a_s;
        if (oacc_out) oacc_out[d] = oacc[d];
    }
}

// ----------------------------------------------------------------------------------------------
// Config 3: prefill GQA attention (composition of SpinQuant_Llama_32_1B/MHA_i8xi8.h:369-427
// with per-head-per-token scales).  q [B,S,HQ,64] s8, qs [B,S,HQ]; k,v [B,S,HKV,64], ks,vs
// [B,S,HKV]; a_s [HQ]; out fp32 [B,S,HQ*64].  Softmax row = the causal prefix 0..t: masked
// entries contribute exactly zero to every partial sum, so the prefix is bit-identical to the
// reference's full padded row.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_mha_prefill(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                             const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                             const float* a_s, int B, int S, int HQ, int HKV, float* out,
                             int8_t* q2_out, float* qs2_out, int8_t* k2_out, float* ks2_out,
                             int32_t* oacc_out) {
    long T = (long)B * S;
    std::vector<int> pos(T);
    for (long t = 0; t < T; t++) pos[t] = (int)(t % S);
    std::vector<int8_t> q2((size_t)T * HQ * 64), k2((size_t)T * HKV * 64);
    std::vector<float> qs2((size_t)T * HQ), ks2((size_t)T * HKV);
    orc_qk_prepare(q, qs, pos.data(), cos_t, sin_t, T, HQ, q2.data(), qs2.data(), nullptr);
    orc_qk_prepare(k, ks, pos.data(), cos_t, sin_t, T, HKV, k2.data(), ks2.data(), nullptr);
    int G = HQ / HKV;
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
    for (int b = 0; b < B; b++)
        for (int t = 0; t < S; t++)
            for (int h = 0; h < HQ; h++) {
                int hk = h / G;
                long qi = ((long)b * S + t) * HQ + h;
                auto at = [&](int j, const int8_t*& kp, float& ksj, const int8_t*& vp, float& vsj) {
                    long ki = ((long)b * S + j) * HKV + hk;
                    kp = k2.data() + ki * 64; ksj = ks2[ki];
                    vp = v + ki * 64; vsj = vs[ki];
                };
                attn_row(q2.data() + qi * 64, qs2[qi], t + 1, at, a_s[h], out + qi * 64,
                         oacc_out ? oacc_out + qi * 64 : nullptr, nullptr, nullptr);
            }
    if (q2_out) std::memcpy(q2_out, q2.data(), q2.size());
    if (qs2_out) std::memcpy(qs2_out, qs2.data(), sizeof(float) * qs2.size());
    if (k2_out) std::memcpy(k2_out, k2.data(), k2.size());
    if (ks2_out) std::memcpy(ks2_out, ks2.data(), sizeof(float) * ks2.size());
}

// ----------------------------------------------------------------------------------------------
// Config 4: one decode step of attention over a paged int8 KV cache, one layer.
// Cache pool: k_pool/v_pool [n_pages][HKV][PAGE][64] s8, ks_pool/vs_pool [n_pages][HKV][PAGE];
// page_table [B][max_pages]; ctx[b] = tokens already cached for sequence b.
// New token: q [B,HQ,64]+qs, k,v [B,HKV,64]+ks,vs. Steps (decode graph order,
// SpinQuant_Decoding_mem_opt.h:1086-1106): RoPE+FHT+requant of q,k at position ctx[b];
// append k,v (cache is MODIFIED); attend over ctx[b]+1 keys.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_mha_decode(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                            const int8_t* v, const float* vs, const float* cos_t, const float* sin_t,
                            const float* a_s, int8_t* k_pool, float* ks_pool, int8_t* v_pool, float* vs_pool,
                            const int32_t* page_table, int max_pages, const int32_t* ctx,
                            int B, int HQ, int HKV, int PAGE, float* out, int32_t* oacc_out) {
    std::vector<int8_t> q2((size_t)B * HQ * 64), k2((size_t)B * HKV * 64);
    std::vector<float> qs2((size_t)B * HQ), ks2((size_t)B * HKV);
    orc_qk_prepare(q, qs, ctx, cos_t, sin_t, B, HQ, q2.data(), qs2.data(), nullptr);
    orc_qk_prepare(k, ks, ctx, cos_t, sin_t, B, HKV, k2.data(), ks2.data(), nullptr);
    for (int b = 0; b < B; b++) {
        int t = ctx[b];
        long pg = page_table[(long)b * max_pages + t / PAGE];
        int slot = t % PAGE;
        for (int h = 0; h < HKV; h++) {
            long row = (pg * HKV + h) * PAGE + slot;
            std::memcpy(k_pool + row * 64, k2.data() + ((long)b * HKV + h) * 64, 64);
            std::memcpy(v_pool + row * 64, v + ((long)b * HKV + h) * 64, 64);
            ks_pool[row] = ks2[(long)b * HKV + h];
            vs_pool[row] = vs[(long)b * HKV + h];
        }
    }
    int G = HQ / HKV;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int b = 0; b < B; b++)
        for (int h = 0; h < HQ; h++) {
            int hk = h / G;
            long qi = (long)b * HQ + h;
            auto at = [&](int j, const int8_t*& kp, float& ksj, const int8_t*& vp, float& vsj) {
                long pg = page_table[(long)b * max_pages + j / PAGE];
                long row = (pg * HKV + hk) * PAGE + (j % PAGE);
                kp = k_pool + row * 64; ksj = ks_pool[row];
                vp = v_pool + row * 64; vsj = vs_pool[row];
            };
            attn_row(q2.data() + qi * 64, qs2[qi], ctx[b] + 1, at, a_s[h], out + qi * 64,
                     oacc_out ? oacc_out + qi * 64 : nullptr, nullptr, nullptr);
        }
}

// Single attention row exposed for fine-grained tests (scores, u8 P, int32 accumulators).
ORC_API void orc_attn_row(const int8_t* q, float qs, const int8_t* k, const float* ks,
                          const int8_t* v, const float* vs, int nk, float a_s,
                          float* out, int32_t* oacc, uint8_t* p, float* score) {
    auto at = [&](int j, const int8_t*& kp, float& ksj, const int8_t*& vp, float& vsj) {
        kp = k + (long)j * 64; ksj = ks[j]; vp = v + (long)j * 64; vsj = vs[j];
    };
    attn_row(q, qs, nk, at, a_s, out, oacc, p, score);
}

// ----------------------------------------------------------------------------------------------
// Config 5: the full quantized Llama-3.2-1B forward (operator order of SpinQuant_Prefilling.h:
// 940-1049 and SpinQuant_Decoding_mem_opt.h:1050-1126, at W8A8 with per-token scales).
//
// Per layer, for the rows of x [M][D] at positions pos[m] of sequence seq[m]:
//   RMSNorm(g0) -> quant -> q,k,v proj -> dequant -> RoPE(q,k) -> FHT-64/8(q,k) -> per-head int8
//   quant of q,k,v -> cache append -> attention (attn_row) -> quant -> o proj -> dequant -> +x
//   -> RMSNorm(g1) -> quant -> gate,up -> dequant -> silu(gate)*up -> FHT-F/sqrt(F) -> quant
//   -> down -> dequant -> +.
// After the last layer: RMSNorm(g_final) -> quant -> lm_head -> dequant -> greedy argmax.
// Embedding row t = (float)lm_head_q[t][:] * lm_head_s[t] (tied embeddings).
// `lanes` selects the RMSNorm order: 0 for prefill, 8 for decode.
// ----------------------------------------------------------------------------------------------
struct OrcModel {
    int L, D, HQ, HKV, F, V;
    float eps, fht_scale;
    const int8_t **wq, **wk, **wv, **wo, **wg, **wu, **wd;
    const float **sq, **sk, **sv, **so, **sg, **su, **sd;
    const float **g0, **g1, **a_s;
    const float* g_final;
    const int8_t* lm_w;
    const float* lm_s;
    const float *cos_t, *sin_t;
};

struct OrcCache {   // contiguous per-sequence cache: [L][B][T][HKV][64]
    int B, T;
    std::vector<int8_t> k, v;
    std::vector<float> ks, vs;
};

static void model_layer(const OrcModel& m, int l, std::vector<float>& x, int M, const int* seq, const int* pos,
                        OrcCache& c, int lanes) {
    const int D = m.D, HQ = m.HQ, HKV = m.HKV, F = m.F, G = HQ / HKV;
    std::vector<float> xn((size_t)M * D), xs(M);
    std::vector<int8_t> xq((size_t)M * D);
    orc_rmsnorm(x.data(), m.g0[l], M, D, m.eps, lanes, xn.data());
    orc_quant_per_token(xn.data(), M, D, xq.data(), xs.data());
    std::vector<float> qf((size_t)M * HQ * 64), kf((size_t)M * HKV * 64), vf((size_t)M * HKV * 64);
    orc_linear_i8(xq.data(), xs.data(), m.wq[l], m.sq[l], M, HQ * 64, D, nullptr, qf.data());
    orc_linear_i8(xq.data(), xs.data(), m.wk[l], m.sk[l], M, HKV * 64, D, nullptr, kf.data());
    orc_linear_i8(xq.data(), xs.data(), m.wv[l], m.sv[l], M, HKV * 64, D, nullptr, vf.data());
    // RoPE + FHT-64 + per-head quant of q and k; per-head quant of v
    std::vector<int8_t> q2((size_t)M * HQ * 64), k2((size_t)M * HKV * 64), v2((size_t)M * HKV * 64);
    std::vector<float> qs2((size_t)M * HQ), ks2((size_t)M * HKV), vs2((size_t)M * HKV);
    auto prep = [&](const float* in, int H, int8_t* out, float* sout, bool rotate) {
#pragma omp parallel for
        for (int t = 0; t < M; t++) {
            const float* cs = m.cos_t + (long)pos[t] * 32;
            const float* sn = m.sin_t + (long)pos[t] * 32;
            for (int h = 0; h < H; h++) {
                long o = ((long)t * H + h) * 64;
                float y[64];
                if (rotate) {
                    for (int k = 0; k < 32; k++) {
                        float x0 = in[o + k], x1 = in[o + k + 32];
                        y[k] = x0 * cs[k] - x1 * sn[k];
                        y[k + 32] = x0 * sn[k] + x1 * cs[k];
                    }
                    fht_inplace(y, 64);
                    for (int k = 0; k < 64; k++) y[k] = y[k] / 8.0f;
                } else {
                    for (int k = 0; k < 64; k++) y[k] = in[o + k];
                }
                float sc = sym_scale(y, 64, 127.0f);
                sout[(long)t * H + h] = sc;
                for (int k = 0; k < 64; k++) out[o + k] = (int8_t)(long long)std::round(y[k] / sc);
            }
        }
    };
    prep(qf.data(), HQ, q2.data(), qs2.data(), true);
    prep(kf.data(), HKV, k2.data(), ks2.data(), true);
    prep(vf.data(), HKV, v2.data(), vs2.data(), false);
    // append to the cache
    const size_t lay = (size_t)l * c.B * c.T;
    for (int t = 0; t < M; t++) {
        size_t row = (lay + (size_t)seq[t] * c.T + pos[t]) * HKV;
        std::memcpy(&c.k[row * 64], &k2[(size_t)t * HKV * 64], (size_t)HKV * 64);
        std::memcpy(&c.v[row * 64], &v2[(size_t)t * HKV * 64], (size_t)HKV * 64);
        std::memcpy(&c.ks[row], &ks2[(size_t)t * HKV], sizeof(float) * HKV);
        std::memcpy(&c.vs[row], &vs2[(size_t)t * HKV], sizeof(float) * HKV);
    }
    std::vector<float> att((size_t)M * HQ * 64);
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int t = 0; t < M; t++)
        for (int h = 0; h < HQ; h++) {
            const int hk = h / G;
            const size_t base = (lay + (size_t)seq[t] * c.T) * HKV;
            auto at = [&](int j, const int8_t*& kp, float& ksj, const int8_t*& vp, float& vsj) {
                size_t row = base + (size_t)j * HKV + hk;
                kp = &c.k[row * 64]; ksj = c.ks[row]; vp = &c.v[row * 64]; vsj = c.vs[row];
            };
            long qi = (long)t * HQ + h;
            attn_row(&q2[qi * 64], qs2[qi], pos[t] + 1, at, m.a_s[l][h], &att[qi * 64], nullptr, nullptr, nullptr);
        }
    std::vector<int8_t> aq((size_t)M * D);
    std::vector<float> as(M), o((size_t)M * D);
    orc_quant_per_token(att.data(), M, D, aq.data(), as.data());
    orc_linear_i8(aq.data(), as.data(), m.wo[l], m.so[l], M, D, D, nullptr, o.data());
    orc_residual(x.data(), o.data(), (long)M * D, x.data());
    std::vector<float> out((size_t)M * D);
    orc_mlp_block(x.data(), m.g1[l], m.wg[l], m.sg[l], m.wu[l], m.su[l], m.wd[l], m.sd[l], M, D, F, m.eps, lanes,
                  m.fht_scale, out.data(), nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    x.swap(out);
}

static void model_embed(const OrcModel& m, const int32_t* tok, int M, std::vector<float>& x) {
    x.resize((size_t)M * m.D);
    for (int t = 0; t < M; t++)
        for (int k = 0; k < m.D; k++) x[(size_t)t * m.D + k] = (float)m.lm_w[(size_t)tok[t] * m.D + k] * m.lm_s[tok[t]];
}

static void model_head(const OrcModel& m, const float* x, int M, int lanes, float* logits, int32_t* next) {
    std::vector<float> xn((size_t)M * m.D), xs(M), lg;
    std::vector<int8_t> xq((size_t)M * m.D);
    orc_rmsnorm(x, m.g_final, M, m.D, m.eps, lanes, xn.data());
    orc_quant_per_token(xn.data(), M, m.D, xq.data(), xs.data());
    if (!logits) { lg.resize((size_t)M * m.V); logits = lg.data(); }
    orc_linear_i8(xq.data(), xs.data(), m.lm_w, m.lm_s, M, m.V, m.D, nullptr, logits);
    if (g_sample_k > 0) orc_topk_sample(logits, M, m.V, g_sample_lanes, g_sample_k, g_sample_rnd + (size_t)g_sample_step * M, next, nullptr, nullptr, nullptr);
    else orc_argmax(logits, M, m.V, next);
}

// tokens [B][S] -> greedy generation of n_new tokens per sequence: out_tokens [B][n_new].
// Optional: hidden_prefill [B*S][D] (residual stream after the last layer), logits_prefill [B][V]
// (last position), logits_last [B][V] (last decode step).
ORC_API void orc_model_generate(const OrcModel* mp, const int32_t* tokens, int B, int S, int n_new,
                                int32_t* out_tokens, float* hidden_prefill, float* logits_prefill, float* logits_last) {
    const OrcModel& m = *mp;
    OrcCache c;
    c.B = B; c.T = S + n_new;
    size_t rows = (size_t)m.L * B * c.T * m.HKV;
    c.k.assign(rows * 64, 0); c.v.assign(rows * 64, 0); c.ks.assign(rows, 0); c.vs.assign(rows, 0);
    const int M = B * S;
    std::vector<int> seq(M), pos(M);
    for (int i = 0; i < M; i++) { seq[i] = i / S; pos[i] = i % S; }
    std::vector<float> x;
    model_embed(m, tokens, M, x);
    for (int l = 0; l < m.L; l++) model_layer(m, l, x, M, seq.data(), pos.data(), c, 0);
    if (hidden_prefill) std::memcpy(hidden_prefill, x.data(), sizeof(float) * x.size());
    std::vector<float> last((size_t)B * m.D);
    for (int b = 0; b < B; b++) std::memcpy(&last[(size_t)b * m.D], &x[((size_t)b * S + S - 1) * m.D], sizeof(float) * m.D);
    std::vector<int32_t> next(B);
    g_sample_step = 0;
    if (n_new <= 0) { if (logits_prefill) model_head(m, last.data(), B, 0, logits_prefill, next.data()); return; }
    model_head(m, last.data(), B, 0, logits_prefill, next.data());
    for (int b = 0; b < B; b++) out_tokens[(size_t)b * n_new] = next[b];
    std::vector<int> dseq(B), dpos(B);
    for (int step = 1; step < n_new; step++) {
        for (int b = 0; b < B; b++) { dseq[b] = b; dpos[b] = S + step - 1; }
        model_embed(m, next.data(), B, x);
        for (int l = 0; l < m.L; l++) model_layer(m, l, x, B, dseq.data(), dpos.data(), c, 8);
        g_sample_step = step;
        model_head(m, x.data(), B, 8, step == n_new - 1 ? logits_last : nullptr, next.data());
        for (int b = 0; b < B; b++) out_tokens[(size_t)b * n_new + step] = next[b];
    }
}

// ----------------------------------------------------------------------------------------------
// HMT (hierarchical memory transformer) plug-in, Modules/HMT.h: the two fp32 primitives of its memory cross-attention.
//
// dec_Linear_Layer_fp32xfp32 (Linear_Layer.h:1040-1101) over PE_fp32xfp32_pack_1x2_1D (PE.h:655-756, the non-versal
// path): y[n] = (p0 + p1) + (p2 + p3), p[c] = sum over k = c, c+4, ... of a[k] * w[n][k], each product and each add
// rounded on its own, k increasing.
// ----------------------------------------------------------------------------------------------
ORC_API void orc_linear_fp32_chain4(const float* a, const float* w, int N, int K, float* y) {
#pragma omp parallel for
    for (int n = 0; n < N; n++) {
        const float* wr = w + (long)n * K;
        float p[4] = {0, 0, 0, 0};
        for (int k = 0; k < K; k++) { const float t = a[k] * wr[k]; p[k & 3] = p[k & 3] + t; }
        const float t0 = p[0] + p[1], t1 = p[2] + p[3];
        y[n] = t0 + t1;
    }
}

// dec_Softmax<float, lanes, dim, enable_scale = true, enable_sub_max = true> (Softmax.h:261-363, non-versal path) as
// hmt_attn_softmax instantiates it (HMT_SpinQuant_Unit.h:97-105): lane i holds elements i * (dim / lanes) + k;
// e = exp((x - max) / scale); per lane four chains over k mod 4, lane total (s0 + s1) + (s2 + s3); lane totals added
// from 0 in lane order; p = e * (1 / total).
ORC_API void orc_softmax_dec(const float* x, int dim, int lanes, float scale, float* pr) {
    const int per = dim / lanes;
    float mx = -1e32f;
    for (int i = 0; i < dim; i++) mx = x[i] > mx ? x[i] : mx;
    float total = 0;
    for (int i = 0; i < lanes; i++) {
        float s[4] = {0, 0, 0, 0};
        for (int k = 0; k < per; k++) {
            const float e = ref_exp((x[i * per + k] - mx) / scale);
            pr[i * per + k] = e;
            s[k & 3] += e;
        }
        total += (s[0] + s[1]) + (s[2] + s[3]);
    }
    const float r = 1.0f / total;
    for (int i = 0; i < dim; i++) pr[i] = pr[i] * r;
}

// One sequence from EMBEDDINGS (HMT feeds the prefill graph vectors that are not rows of the embedding table): prefill of
// S rows (positions 0 .. S-1; rows from n_valid on are padding), residual stream out [S][D]; then greedy generation of n_new
// tokens continuing after position n_valid - 1.
ORC_API void orc_model_forward_embeds(const OrcModel* mp, const float* embeds, int S, int n_valid, int n_new, float* hidden_out,
                                      int32_t* out_tokens) {
    const OrcModel& m = *mp;
    OrcCache c;
    c.B = 1; c.T = S + (n_new > 0 ? n_new : 0);
    size_t rows = (size_t)m.L * c.T * m.HKV;
    c.k.assign(rows * 64, 0); c.v.assign(rows * 64, 0); c.ks.assign(rows, 0); c.vs.assign(rows, 0);
    std::vector<int> seq(S, 0), pos(S);
    for (int i = 0; i < S; i++) pos[i] = i;
    std::vector<float> x(embeds, embeds + (size_t)S * m.D);
    for (int l = 0; l < m.L; l++) model_layer(m, l, x, S, seq.data(), pos.data(), c, 0);
    if (hidden_out) std::memcpy(hidden_out, x.data(), sizeof(float) * x.size());
    if (n_new <= 0) return;
    std::vector<float> last(&x[(size_t)(n_valid - 1) * m.D], &x[(size_t)n_valid * m.D]);
    int32_t next = 0;
    g_sample_step = 0;
    model_head(m, last.data(), 1, 0, nullptr, &next);
    out_tokens[0] = next;
    for (int step = 1; step < n_new; step++) {
        int dseq = 0, dpos = n_valid + step - 1;
        model_embed(m, &next, 1, x);
        for (int l = 0; l < m.L; l++) model_layer(m, l, x, 1, &dseq, &dpos, c, 8);
        g_sample_step = step;
        model_head(m, x.data(), 1, 8, nullptr, &next);
        out_tokens[step] = next;
    }
}

