// Tier-A oracle: the reference's OWN operator templates (FlexLLM `Modules/*.h`), compiled
// unmodified from where they lie (-I <reference>/Modules) against the stand-in headers in
// oracle/ref_shim, and exported through a small C API so that tests can run them.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is used to pin the plain-C++ restatement
// (oracle/flexllm_oracle.cpp) and to generate the fixtures under tests/golden/. The product
// library never links or loads it. Output goes to oracle/_ref/libflexllm_ref.so only.
//
// Each wrapper fills the input streams in the order the reference's loaders produce
// (token-parallel vectors for pref_*, block-partitioned lanes for dec_*), calls the template,
// and drains the output stream back into a row-major array.

#include <iostream>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <vector>
#include <cstdint>

// The operator templates print progress lines from inside their loops; swallow them.
struct orc_null_sink {
    template <class T> orc_null_sink& operator<<(const T&) { return *this; }
    orc_null_sink& operator<<(std::ostream& (*)(std::ostream&)) { return *this; }
};
static orc_null_sink orc_sink;
#define cout orc_sink
#define printf(...) ((void)0)

#include "config.h"
#include "PE.h"
#include "data_io.h"
#include "quant.h"
#include "FHT.h"
#include "RoPE.h"
#include "Softmax.h"
#include "LayerNorm.h"
#include "Swish.h"
#include "Residual_Layer.h"
#include "Logits.h"
#include "Linear_Layer.h"
#include "MHA.h"

#undef cout
#undef printf

#define REF_API extern "C" __attribute__((visibility("default")))

using fvec1 = hls::vector<float, 1>;

// ---- quant.h:6 pref_quant_layer_fp32_qint<8,false,...> -----------------------------------------
REF_API void ref_quant_per_token(const float* x, int M, int K, int8_t* q, float* s) {
    constexpr int P = 8;
    static_assert(P == 8, "");
    for (int m0 = 0; m0 < M; m0 += P) {
        tapa::stream<hls::vector<float, P>> in;
        tapa::stream<hls::vector<float, 1>> sb;
        tapa::stream<hls::vector<ap_int<8>, P>> out;
        for (int k = 0; k < K; k++) {
            hls::vector<float, P> v;
            for (int m = 0; m < P; m++) v[m] = (m0 + m < M) ? x[(long)(m0 + m) * K + k] : 0.0f;
            in.write(v);
        }
        pref_quant_layer_fp32_qint<8, false, P, 8192, P>(in, sb, out, P, K);
        for (int m = 0; m < P; m++) { float sc = sb.read()[0]; if (m0 + m < M) s[m0 + m] = sc; }
        for (int k = 0; k < K; k++) {
            auto v = out.read();
            for (int m = 0; m < P; m++) if (m0 + m < M) q[(long)(m0 + m) * K + k] = (int8_t)(long long)v[m];
        }
    }
}

// ---- quant.h:333 dec_quant_layer_fp32_qint<8,false,BP,...>: one token, BP block lanes ----------
REF_API void ref_dec_quant_per_token(const float* x, int M, int K, int8_t* q, float* s) {
    constexpr int BP = 8;
    for (int m = 0; m < M; m++) {
        tapa::stream<hls::vector<float, BP>> in;
        tapa::stream<hls::vector<float, 1>> sb;
        tapa::stream<hls::vector<ap_int<8>, BP>> out;
        const float* xr = x + (long)m * K;
        for (int i = 0; i < K / BP; i++) {
            hls::vector<float, BP> v;
            for (int l = 0; l < BP; l++) v[l] = xr[l * (K / BP) + i];
            in.write(v);
        }
        dec_quant_layer_fp32_qint<8, false, BP, 8192>(in, sb, out, K);
        s[m] = sb.read()[0];
        for (int i = 0; i < K / BP; i++) {
            auto v = out.read();
            for (int l = 0; l < BP; l++) q[(long)m * K + l * (K / BP) + i] = (int8_t)(long long)v[l];
        }
    }
}

// ---- quant.h:116 pref_dequant_layer_qint_fp32<32,false,...> ------------------------------------
REF_API void ref_dequant(const int32_t* acc, const float* s_tok, const float* s_ch, int M, int N, float* y) {
    constexpr int P = 1;
    for (int m = 0; m < M; m++) {
        tapa::stream<hls::vector<ap_int<32>, P>> in;
        tapa::stream<hls::vector<float, 1>> sb, ws;
        tapa::stream<hls::vector<float, P>> out;
        sb.write(fvec1(s_tok[m]));
        for (int n = 0; n < N; n++) {
            hls::vector<ap_int<32>, P> v; v[0] = ap_int<32>(acc[(long)m * N + n]);
            in.write(v);
            ws.write(fvec1(s_ch[n]));
        }
        pref_dequant_layer_qint_fp32<32, false, P, 8192, 1>(in, sb, ws, out, 1, N);
        for (int n = 0; n < N; n++) y[(long)m * N + n] = out.read()[0];
    }
}

// ---- quant.h:6 pref_quant_layer_fp32_qint<4,true,...>: the shipped model's activation quantiser (4-bit asymmetric) ----
REF_API void ref_quant_per_token_asym4(const float* x, int M, int K, uint8_t* q, float* s, float* b) {
    constexpr int P = 8;
    for (int m0 = 0; m0 < M; m0 += P) {
        tapa::stream<hls::vector<float, P>> in;
        tapa::stream<hls::vector<float, 2>> sb;
        tapa::stream<hls::vector<ap_int<4>, P>> out;
        for (int k = 0; k < K; k++) {
            hls::vector<float, P> v;
            for (int m = 0; m < P; m++) v[m] = (m0 + m < M) ? x[(long)(m0 + m) * K + k] : 0.0f;
            in.write(v);
        }
        pref_quant_layer_fp32_qint<4, true, P, 8192, P>(in, sb, out, P, K);
        for (int m = 0; m < P; m++) { auto t = sb.read(); if (m0 + m < M) { s[m0 + m] = t[0]; b[m0 + m] = t[1]; } }
        for (int k = 0; k < K; k++) {
            auto v = out.read();
            for (int m = 0; m < P; m++) if (m0 + m < M) q[(long)(m0 + m) * K + k] = (uint8_t)((long long)v[m] & 15);   // the 4 bits, read as unsigned
        }
    }
}

// ---- quant.h:116 pref_dequant_layer_qint_fp32<.., true, ..>: acc * s * ws + b * wsum ---------------------------------
REF_API void ref_dequant_asym(const int32_t* acc, const float* s_tok, const float* b_tok, const float* s_ch, const float* wsum, int M,
                              int N, float* y) {
    constexpr int P = 1;
    for (int m = 0; m < M; m++) {
        tapa::stream<hls::vector<ap_int<32>, P>> in;
        tapa::stream<hls::vector<float, 2>> sb, ws;
        tapa::stream<hls::vector<float, P>> out;
        hls::vector<float, 2> t; t[0] = s_tok[m]; t[1] = b_tok[m];
        sb.write(t);
        for (int n = 0; n < N; n++) {
            hls::vector<ap_int<32>, P> v; v[0] = ap_int<32>(acc[(long)m * N + n]);
            in.write(v);
            hls::vector<float, 2> u; u[0] = s_ch[n]; u[1] = wsum[n];
            ws.write(u);
        }
        pref_dequant_layer_qint_fp32<32, true, P, 8192, 1>(in, sb, ws, out, 1, N);
        for (int n = 0; n < N; n++) y[(long)m * N + n] = out.read()[0];
    }
}

// ---- Linear_Layer.h:9 systolic_array_i4xi4_pack_2x2_2D<.., is_uint_A = true>: unsigned 4-bit activations x signed 4-bit weights ----
REF_API void ref_gemm_u4s4(const uint8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
    constexpr int BA = 8, BB = 16, LOG2K = 13;
    for (int m0 = 0; m0 < M; m0 += BA)
        for (int n0 = 0; n0 < N; n0 += BB) {
            hls::stream<hls::vector<ap_int<4>, BA>> A;
            hls::stream<hls::vector<ap_int<4>, BB>> B;
            hls::stream<hls::vector<ap_int<LOG2K + 8>, BA>> C;
            for (int k = 0; k < K; k++) {
                hls::vector<ap_int<4>, BA> va;
                hls::vector<ap_int<4>, BB> vb;
                for (int i = 0; i < BA; i++) va[i] = ap_int<4>((int)((m0 + i < M) ? a[(long)(m0 + i) * K + k] : 0));
                for (int j = 0; j < BB; j++) vb[j] = ap_int<4>((int)((n0 + j < N) ? w[(long)(n0 + j) * K + k] : 0));
                A.write(va);
                B.write(vb);
            }
            systolic_array_i4xi4_pack_2x2_2D<BA, BB, LOG2K, true>(A, B, C, K);
            for (int j = 0; j < BB; j++) {
                auto c = C.read();
                for (int i = 0; i < BA; i++)
                    if (m0 + i < M && n0 + j < N) acc[(long)(m0 + i) * N + n0 + j] = (int32_t)(long long)c[i];
            }
        }
}

// ---- MHA.h:114 systolic_array_i8xi8_pack_2x2 (s8 x s8 and u8 x s8), tiled 8 x 16 ---------------
template <bool is_uint_A>
static void ref_gemm(const int8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
    constexpr int BA = 8, BB = 16, LOG2K = 13;
    for (int m0 = 0; m0 < M; m0 += BA)
        for (int n0 = 0; n0 < N; n0 += BB) {
            hls::stream<hls::vector<ap_int<8>, BA>> A;
            hls::stream<hls::vector<ap_int<8>, BB>> B;
            hls::stream<hls::vector<ap_int<LOG2K + 16>, BA>> C;
            for (int k = 0; k < K; k++) {
                hls::vector<ap_int<8>, BA> va;
                hls::vector<ap_int<8>, BB> vb;
                for (int i = 0; i < BA; i++) va[i] = ap_int<8>((int)((m0 + i < M) ? a[(long)(m0 + i) * K + k] : 0));
                for (int j = 0; j < BB; j++) vb[j] = ap_int<8>((int)((n0 + j < N) ? w[(long)(n0 + j) * K + k] : 0));
                A.write(va);
                B.write(vb);
            }
            systolic_array_i8xi8_pack_2x2<BA, BB, LOG2K, is_uint_A>(A, B, C, K);
            for (int j = 0; j < BB; j++) {
                auto c = C.read();
                for (int i = 0; i < BA; i++)
                    if (m0 + i < M && n0 + j < N) acc[(long)(m0 + i) * N + n0 + j] = (int32_t)(long long)c[i];
            }
        }
}
REF_API void ref_gemm_s8s8(const int8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
    ref_gemm<false>(a, w, M, N, K, acc);
}
REF_API void ref_gemm_u8s8(const uint8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
    ref_gemm<true>((const int8_t*)a, w, M, N, K, acc);
}

// ---- FHT.h:8 pref_FHT and FHT.h:70 dec_FHT -----------------------------------------------------
template <int N, int LOG2N>
static void ref_fht_n(const float* x, long rows, float scale, float* y) {
    for (long r = 0; r < rows; r++) {
        tapa::stream<fvec1> in, out;
        for (int k = 0; k < N; k++) in.write(fvec1(x[r * N + k]));
        pref_FHT<float, 1, N, LOG2N, 1>(in, out, 1, scale);
        for (int k = 0; k < N; k++) y[r * N + k] = out.read()[0];
    }
}
REF_API int ref_fht(const float* x, long rows, int N, float scale, float* y) {
    if (N == 64) ref_fht_n<64, 6>(x, rows, scale, y);
    else if (N == 256) ref_fht_n<256, 8>(x, rows, scale, y);
    else if (N == 8192) ref_fht_n<8192, 13>(x, rows, scale, y);
    else return -1;
    return 0;
}
REF_API int ref_dec_fht(const float* x, long rows, int N, float scale, float* y) {
    if (N != 8192) return -1;
    constexpr int BP = 16, NN = 8192;
    for (long r = 0; r < rows; r++) {
        tapa::stream<hls::vector<float, BP>> in, out;
        for (int i = 0; i < NN / BP; i++) {
            hls::vector<float, BP> v;
            for (int l = 0; l < BP; l++) v[l] = x[r * NN + l * (NN / BP) + i];
            in.write(v);
        }
        dec_FHT<float, BP, NN, 13>(in, out, scale);
        for (int i = 0; i < NN / BP; i++) {
            auto v = out.read();
            for (int l = 0; l < BP; l++) y[r * NN + l * (NN / BP) + i] = v[l];
        }
    }
    return 0;
}

// ---- RoPE.h:9 pref_RoPE_layer (positions 0..S-1) and RoPE.h:97 dec_RoPE_layer -------------------
// x, y: [S][H][64]; tables [>=S][32]
REF_API int ref_rope_prefill(const float* x, const float* cos_t, const float* sin_t, int S, int H, float* y) {
    constexpr int MAXS = 1024;
    if (S > MAXS) return -1;
    static float PS[MAXS][32], PC[MAXS][32];
    std::memcpy(PS, sin_t, sizeof(float) * S * 32);
    std::memcpy(PC, cos_t, sizeof(float) * S * 32);
    tapa::stream<fvec1> in, out;
    for (int t = 0; t < S; t++)
        for (int h = 0; h < H; h++)
            for (int k = 0; k < 64; k++) in.write(fvec1(x[((long)t * H + h) * 64 + k]));
    pref_RoPE_layer<float, 1, 64, 32, MAXS>(in, out, PS, PC, H, S);
    for (int t = 0; t < S; t++)
        for (int h = 0; h < H; h++)
            for (int k = 0; k < 64; k++) y[((long)t * H + h) * 64 + k] = out.read()[0];
    return 0;
}
// one token at position pos; x, y: [H][64]
REF_API int ref_rope_decode(const float* x, const float* cos_t, const float* sin_t, int P, int pos, int H, float* y) {
    constexpr int MAXS = 8448;
    if (P > MAXS || pos >= P) return -1;
    static float PS[MAXS][32], PC[MAXS][32];
    std::memcpy(PS, sin_t, sizeof(float) * (size_t)P * 32);
    std::memcpy(PC, cos_t, sizeof(float) * (size_t)P * 32);
    tapa::stream<fvec1> in, out;
    for (int h = 0; h < H; h++)
        for (int k = 0; k < 64; k++) in.write(fvec1(x[h * 64 + k]));
    dec_RoPE_layer<float, 1, 64, 32, MAXS>(in, out, PS, PC, H, pos);
    for (int h = 0; h < H; h++)
        for (int k = 0; k < 64; k++) y[h * 64 + k] = out.read()[0];
    return 0;
}

// ---- MHA.h:247 pref_causal_mask_template + Softmax.h:7 pref_Softmax ------------------------------
// x: [S][len] score rows of one head; causal != 0 applies the mask (row t keeps k <= t).
REF_API int ref_softmax_prefill(const float* x, int S, int len, int causal, float* p) {
    constexpr int MAXL = 8192;
    if (len > MAXL || (len & 3)) return -1;
    for (int t = 0; t < S; t++) {
        tapa::stream<fvec1> in, mid, out;
        for (int k = 0; k < len; k++) in.write(fvec1(x[(long)t * len + k]));
        if (causal) {
            // the mask template derives the query index from its own block counter, so feed it
            // t+1 rows and keep the last one
            tapa::stream<fvec1> in2, mid2;
            for (int r = 0; r <= t; r++)
                for (int k = 0; k < len; k++) in2.write(fvec1(x[(long)t * len + k]));
            pref_causal_mask_template<float, 1, MAXL, 1, 1>(in2, mid2, t + 1, len);
            for (int r = 0; r < t; r++) for (int k = 0; k < len; k++) mid2.read();
            for (int k = 0; k < len; k++) mid.write(mid2.read());
            pref_Softmax<float, 1, MAXL, 1, 1>(mid, out, 1, len);
        } else {
            pref_Softmax<float, 1, MAXL, 1, 1>(in, out, 1, len);
        }
        for (int k = 0; k < len; k++) p[(long)t * len + k] = out.read()[0];
    }
    return 0;
}
// ---- Softmax.h:457 dec_MHA_Softmax: rows of arbitrary length ------------------------------------
REF_API int ref_softmax_decode(const float* x, int len, float* p) {
    constexpr int MAXL = 8448;
    if (len > MAXL) return -1;
    tapa::stream<fvec1> in, out;
    for (int k = 0; k < len; k++) in.write(fvec1(x[k]));
    dec_MHA_Softmax<float, 1, MAXL, 1>(in, out, len);
    for (int k = 0; k < len; k++) p[k] = out.read()[0];
    return 0;
}

// ---- LayerNorm.h:29 pref_Layer_Norm / :211 dec_Layer_Norm ---------------------------------------
REF_API void ref_rmsnorm_prefill(const float* x, const float* gamma, int M, int D, float* y) {
    for (int m = 0; m < M; m++) {
        tapa::stream<fvec1> in, out;
        tapa::stream<float> g;
        for (int k = 0; k < D; k++) { in.write(fvec1(x[(long)m * D + k])); g.write(gamma[k]); }
        pref_Layer_Norm<float, 1, 8192, 1>(in, g, out, 1, D);
        for (int k = 0; k < D; k++) y[(long)m * D + k] = out.read()[0];
    }
}
template <int BP>
static void ref_rmsnorm_dec(const float* x, const float* gamma, int M, int D, float* y) {
    for (int m = 0; m < M; m++) {
        tapa::stream<hls::vector<float, BP>> in, g, out;
        for (int i = 0; i < D / BP; i++) {
            hls::vector<float, BP> v, w;
            for (int l = 0; l < BP; l++) { v[l] = x[(long)m * D + l * (D / BP) + i]; w[l] = gamma[l * (D / BP) + i]; }
            in.write(v); g.write(w);
        }
        dec_Layer_Norm<float, BP, 8192>(in, g, out, D);
        for (int i = 0; i < D / BP; i++) {
            auto v = out.read();
            for (int l = 0; l < BP; l++) y[(long)m * D + l * (D / BP) + i] = v[l];
        }
    }
}
REF_API int ref_rmsnorm_decode(const float* x, const float* gamma, int M, int D, int lanes, float* y) {
    if (lanes == 4) ref_rmsnorm_dec<4>(x, gamma, M, D, y);
    else if (lanes == 8) ref_rmsnorm_dec<8>(x, gamma, M, D, y);
    else return -1;
    return 0;
}

// ---- Swish.h:6, Linear_Layer.h:613, Residual_Layer.h:47 -----------------------------------------
REF_API void ref_silu(const float* g, long n, float* y) {
    tapa::stream<fvec1> in, out;
    for (long i = 0; i < n; i++) in.write(fvec1(g[i]));
    pref_Swish<float, 1, 1, 1>(in, out, (int)n, 1);
    for (long i = 0; i < n; i++) y[i] = out.read()[0];
}
REF_API void ref_gate_mul(const float* a, const float* b, long n, float* y) {
    tapa::stream<fvec1> in, gt, out;
    for (long i = 0; i < n; i++) { in.write(fvec1(a[i])); gt.write(fvec1(b[i])); }
    pref_Gate_Layer_fp32xfp32<1, 1, 1>(in, gt, out, (int)n);
    for (long i = 0; i < n; i++) y[i] = out.read()[0];
}
REF_API void ref_residual(const float* a, const float* b, long n, float* y) {
    tapa::stream<fvec1> in, rs, out;
    for (long i = 0; i < n; i++) { in.write(fvec1(a[i])); rs.write(fvec1(b[i])); }
    pref_Residual_Layer<float, 1, 1, 1>(in, rs, out, (int)n);
    for (long i = 0; i < n; i++) y[i] = out.read()[0];
}

// ---- quant.h:253 pref_static_sym_per_tensor_quant_layer_fp32_qint (signed and unsigned) --------
// x: [rows][n]; one scale s (table [16][1] filled with s); f = mha_scale_factor.
template <int is_signed>
static void ref_static_q(const float* x, long rows, int n, float s, float f, uint8_t* q) {
    static float tab[DECODER_LAYER_NUM][1];
    for (auto& r : tab) r[0] = s;
    tapa::stream<fvec1> in;
    tapa::stream<hls::vector<ap_int<8>, 1>> out;
    for (long i = 0; i < rows * n; i++) in.write(fvec1(x[i]));
    pref_static_sym_per_tensor_quant_layer_fp32_qint<8, 1, 8192, 1, is_signed, 1>(in, out, tab, 0, (int)rows, n, f);
    for (long i = 0; i < rows * n; i++) q[i] = (uint8_t)(long long)out.read()[0];
}
REF_API void ref_static_quant(const float* x, long rows, int n, float s, float f, int is_signed, uint8_t* q) {
    if (is_signed) ref_static_q<1>(x, rows, n, s, f, q); else ref_static_q<0>(x, rows, n, s, f, q);
}

// ---- quant.h:167 pref_static_sym_quant_layer_fp32_qint: per-token scale stream ------------------
REF_API void ref_scale_stream_quant(const float* x, long rows, int n, const float* s, int is_signed, uint8_t* q) {
    tapa::stream<fvec1> in, sc;
    tapa::stream<hls::vector<ap_int<8>, 1>> out;
    for (long r = 0; r < rows; r++) {
        sc.write(fvec1(s[r]));
        for (int k = 0; k < n; k++) in.write(fvec1(x[r * n + k]));
    }
    if (is_signed) pref_static_sym_quant_layer_fp32_qint<8, 1, 1, 8192, 1, true, 1>(in, sc, out, (int)rows, n);
    else pref_static_sym_quant_layer_fp32_qint<8, 1, 1, 8192, 1, false, 1>(in, sc, out, (int)rows, n);
    for (long i = 0; i < rows * n; i++) q[i] = (uint8_t)(long long)out.read()[0];
}

// ---- quant.h:214 pref_static_sym_dequant_layer_qint_fp32: score = acc * s_q[m] * s_k[n] --------
REF_API void ref_scale_stream_dequant(const int32_t* acc, const float* s_row, const float* s_col,
                                      int M, int N, float* y) {
    for (int m = 0; m < M; m++) {
        tapa::stream<hls::vector<ap_int<32>, 1>> in;
        tapa::stream<fvec1> sr, out;
        tapa::stream<float> scs;
        sr.write(fvec1(s_row[m]));
        for (int n = 0; n < N; n++) {
            hls::vector<ap_int<32>, 1> v; v[0] = ap_int<32>(acc[(long)m * N + n]);
            in.write(v);
            scs.write(s_col[n]);
        }
        pref_static_sym_dequant_layer_qint_fp32<32, 1, 1, 8192, 1, 1, 1>(in, sr, scs, out, 1, N);
        for (int n = 0; n < N; n++) y[(long)m * N + n] = out.read()[0];
    }
}

// ---- quant.h:528 dec_MHA_quant_layer_fp32_qint: per-head dynamic quant, head_dim 64 -------------
// x: [H][64] -> q [H][64], s [H]
REF_API void ref_head_quant(const float* x, int H, int8_t* q, float* s) {
    for (int h = 0; h < H; h++) {
        tapa::stream<fvec1> in;
        tapa::stream<hls::vector<float, 1>> sb;
        tapa::stream<hls::vector<ap_int<8>, 1>> out;
        for (int k = 0; k < 64; k++) in.write(fvec1(x[h * 64 + k]));
        dec_MHA_quant_layer_fp32_qint<8, false, 1, 64, 1>(in, sb, out, 64);
        s[h] = sb.read()[0];
        for (int k = 0; k < 64; k++) q[h * 64 + k] = (int8_t)(long long)out.read()[0];
    }
}

// ---- MHA.h:190 pref_MHA_i8xi8_qxk_template: S x S integer scores of G query heads vs one KV head
// q: [S][G][64], k: [S][64] -> acc [S][G][S]   (S multiple of 16)
REF_API int ref_mha_qxk(const int8_t* q, const int8_t* k, int S, int G, int32_t* acc) {
    constexpr int P = 8, KP = 16, MAXS = 1024;
    if (S % KP || S > MAXS || G != 4) return -1;
    tapa::stream<hls::vector<ap_int<8>, P>> qs;
    tapa::stream<hls::vector<ap_int<8>, KP>> ks;
    tapa::stream<hls::vector<ap_int<22>, P>> os;
    for (int M = 0; M < S / P; M++)
        for (int h = 0; h < G; h++) {
            for (int d = 0; d < 64; d++) {
                hls::vector<ap_int<8>, P> v;
                for (int m = 0; m < P; m++) v[m] = ap_int<8>((int)q[((long)(M * P + m) * G + h) * 64 + d]);
                qs.write(v);
            }
            for (int N = 0; N < S / KP; N++)
                for (int d = 0; d < 64; d++) {
                    hls::vector<ap_int<8>, KP> v;
                    for (int n = 0; n < KP; n++) v[n] = ap_int<8>((int)k[(long)(N * KP + n) * 64 + d]);
                    ks.write(v);
                }
        }
    pref_MHA_i8xi8_qxk_template<P, KP, 4, 64, 6, MAXS>(qs, ks, os, S);
    for (int M = 0; M < S / P; M++)
        for (int h = 0; h < G; h++)
            for (int j = 0; j < S; j++) {
                auto c = os.read();
                for (int m = 0; m < P; m++) acc[((long)(M * P + m) * G + h) * S + j] = (int32_t)(long long)c[m];
            }
    return 0;
}

// ---- MHA.h:340 pref_MHA_i8xi8_axv_template (unsigned P): out[S][G][64] = sum_j p[S][G][j] v[j][64]
REF_API int ref_mha_axv(const uint8_t* p, const int8_t* v, int S, int G, int32_t* acc) {
    constexpr int P = 8, VP = 16, MAXS = 1024;
    if (S % P || S > MAXS || G != 4) return -1;
    tapa::stream<hls::vector<ap_int<8>, P>> ps;
    tapa::stream<hls::vector<ap_int<8>, VP>> vs;
    tapa::stream<hls::vector<ap_int<26>, P>> os;
    for (int M = 0; M < S / P; M++)
        for (int h = 0; h < G; h++) {
            for (int j = 0; j < S; j++) {
                hls::vector<ap_int<8>, P> a;
                for (int m = 0; m < P; m++) a[m] = ap_int<8>((int)p[((long)(M * P + m) * G + h) * S + j]);
                ps.write(a);
            }
            for (int N = 0; N < 64 / VP; N++)
                for (int j = 0; j < S; j++) {
                    hls::vector<ap_int<8>, VP> b;
                    for (int n = 0; n < VP; n++) b[n] = ap_int<8>((int)v[(long)j * 64 + N * VP + n]);
                    vs.write(b);
                }
        }
    pref_MHA_i8xi8_axv_template<P, VP, 4, 64, MAXS, 10, true>(ps, vs, os, S);
    for (int M = 0; M < S / P; M++)
        for (int h = 0; h < G; h++)
            for (int d = 0; d < 64; d++) {
                auto c = os.read();
                for (int m = 0; m < P; m++) acc[((long)(M * P + m) * G + h) * 64 + d] = (int32_t)(long long)c[m];
            }
    return 0;
}

// ---- Logits.h:6 sort_top_k: greedy token = rank 0 after inserting every logit in index order -----
REF_API void ref_argmax(const float* logits, int B, long V, int32_t* idx) {
    for (int b = 0; b < B; b++) {
        constexpr int TOPK = 5;  // LOGITS_MAX_K in the accelerator configs
        int ids[TOPK];
        float vals[TOPK];
        for (int k = 0; k < TOPK; k++) { ids[k] = -1; vals[k] = -INFINITY; }
        for (long v = 0; v < V; v++) sort_top_k<float, TOPK>(ids, vals, (int)v, logits[(long)b * V + v]);
        idx[b] = ids[0];
    }
}

// ---- Logits.h:145-279 dec_Sampling_Embedding_Layer: per-lane top-k, merge, softmax over k, inverse-CDF
// sample from a host-supplied uniform number. Instantiated like the decode graphs do it
// (SpinQuant_Llama_32_1B/SpinQuant_Decoding_mem_opt.h:934: top_k = 5, inner_block_parallel = 1,
// enable_sub_max) with P = 16 or 32 lanes; the embedding gather that follows reads a dummy table.
template <int P>
static int ref_topk_sample_p(const float* logits, int V, float rnd, int32_t* idx) {
    constexpr int MAXV = 1 << 17, HID = 64, BPE = 16;
    if (V > MAXV || V % P) return -1;
    tapa::stream<hls::vector<float, P>> ls;
    for (int t = 0; t < V / P; t++) {
        hls::vector<float, P> v;
        for (int i = 0; i < P; i++) v[i] = logits[(long)i * (V / P) + t];
        ls.write(v);
    }
    std::vector<hls::vector<float, BPE>> vocab((size_t)V * HID / BPE);
    tapa::mmap<hls::vector<float, BPE>> vm(vocab.data());
    tapa::stream<hls::vector<float, BPE>> es;
    int sampled = -1;
    dec_Sampling_Embedding_Layer<float, P, MAXV, 5, BPE, HID, P * 8>(ls, vm, es, rnd, sampled, V, HID);
    for (int i = 0; i < HID / BPE; i++) (void)es.read();
    *idx = sampled;
    return 0;
}
REF_API int ref_topk_sample(const float* logits, int V, int lanes, float rnd, int32_t* idx) {
    if (lanes == 16) return ref_topk_sample_p<16>(logits, V, rnd, idx);
    if (lanes == 32) return ref_topk_sample_p<32>(logits, V, rnd, idx);
    return -1;
}

// ---- Linear_Layer.h:1040 dec_Linear_Layer_fp32xfp32<4, 8, ...> (the HMT cross-attention's linear unit) -------------------
// One input vector x [K] against W [N][K]. Lanes are block-partitioned: lane i carries inputs i * K/4 + k and produces the
// outputs i * N/4 + ...; each lane's weight stream delivers, for its output block, 8 rows at a time, column by column in the
// order the layer replays the input (lane blocks 0..3, k inside the block).
REF_API int ref_linear_fp32(const float* x, const float* w, int N, int K, float* y) {
    constexpr int BP = 4, WP = 8, MAXD = 2048;
    if (K % (BP * 4) || N % (BP * WP) || K > MAXD || N > MAXD) return -1;
    tapa::stream<hls::vector<float, BP>> in, out;
    tapa::stream<hls::vector<float, WP>> wls[BP];
    tapa::istreams<hls::vector<float, WP>, BP> wl;
    for (int i = 0; i < BP; i++) wl.s[i] = &wls[i];
    // dec_Linear_Layer_fp32xfp32 stores A[i * MAXD/BP + k] = pack[i] and replays A[Kb * MAXD/BP + k]: feed K == MAXD-shaped input
    // by placing element i * (K/BP) + k in lane i at position k only when K == MAXD; for smaller K the same holds because the
    // replay uses the same (lane block, k) addressing.
    for (int k = 0; k < K / BP; k++) {
        hls::vector<float, BP> v;
        for (int i = 0; i < BP; i++) v[i] = x[i * (K / BP) + k];
        in.write(v);
    }
    for (int Nb = 0; Nb < N / (BP * WP); Nb++)
        for (int Kb = 0; Kb < BP; Kb++)
            for (int k = 0; k < K / BP; k++)
                for (int i = 0; i < BP; i++) {
                    hls::vector<float, WP> wv;
                    for (int n = 0; n < WP; n++) wv[n] = w[(long)(i * (N / BP) + Nb * WP + n) * K + Kb * (K / BP) + k];
                    wls[i].write(wv);
                }
    dec_Linear_Layer_fp32xfp32<BP, WP, MAXD, MAXD>(in, wl, out, K, N);
    for (int Nb = 0; Nb < N / (BP * WP); Nb++)
        for (int n = 0; n < WP; n++) {
            auto v = out.read();
            for (int i = 0; i < BP; i++) y[i * (N / BP) + Nb * WP + n] = v[i];
        }
    return 0;
}

// ---- Softmax.h:261 dec_Softmax<float, 4, 64, true, true> as hmt_attn_softmax instantiates it -------------------------------
REF_API int ref_softmax_dec4_64(const float* x, float scale, float* p) {
    constexpr int BP = 4, DIM = 64;
    tapa::stream<hls::vector<float, BP>> in, out;
    for (int k = 0; k < DIM / BP; k++) {
        hls::vector<float, BP> v;
        for (int i = 0; i < BP; i++) v[i] = x[i * (DIM / BP) + k];
        in.write(v);
    }
    dec_Softmax<float, BP, DIM, true, true>(in, out, DIM, scale);
    for (int k = 0; k < DIM / BP; k++) {
        auto v = out.read();
        for (int i = 0; i < BP; i++) p[i * (DIM / BP) + k] = v[i];
    }
    return 0;
}

