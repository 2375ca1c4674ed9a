// Reader for the reference's on-disk model format (host code only).
//
// The FlexLLM demo keeps a SpinQuant-exported Llama-3.2-1B under parameters/ in two kinds of files
// (SpinQuant_Llama_32_1B_Ins/SpinQuant_Prefilling_Decoding_mem_opt_demo.cpp:21-74, :132-175, :437-490):
//   <proj>_L%02d.bin             int8, row-major [out][in], one byte per weight (values in [-8, 7] for the shipped 4-bit
//                                model; any int8 is accepted here), proj in {q,k,v,o,gate,up,down}_proj, plus lm_head_L00.bin
//   model_embed_tokens_fp32.bin  fp32 [vocab][hidden]
//   *.h                          C array definitions that the demo #includes: w_<proj>_s[layers][out] and
//                                w_<proj>_sum[layers][out] in w_<proj>_s_sum.h (per-channel scale, and the row sums
//                                sum_k w[n][k] * s[n] of the asymmetric dequantiser), RMSNorm_weight[2*layers+1][hidden]
//                                in w_rmsnorm.h, A_s[layers][heads_q] in A_s.h, PE_sin / PE_cos[pos][32] in
//                                RoPE_sin_cos.h, w_lm_head_lm_head_s[vocab] / _sum[vocab] in w_lm_head_lm_head.h
// The demo re-packs the .bin rows two 4-bit channels per byte into its FPGA lane layout while reading; here rows are
// kept as int8 [out][in], the layout every linear layer of this library takes.
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace flexllm {

static bool slurp(const std::string& path, std::string* out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    out->resize(n > 0 ? (size_t)n : 0);
    const size_t got = n > 0 ? fread(&(*out)[0], 1, (size_t)n, f) : 0;
    fclose(f);
    return got == out->size();
}

// Parses `count` numbers of the initialiser of the C array `name` in `text`, skipping the first `skip` numbers.
// Accepts nested braces, float suffixes and // or /* */ comments. Returns the numbers read (< count: too few).
static long parse_c_array(const std::string& text, const char* name, long skip, long count, float* out) {
    const size_t len = strlen(name);
    size_t pos = 0;
    for (;;) {
        pos = text.find(name, pos);
        if (pos == std::string::npos) return -1;
        const bool left_ok = pos == 0 || !(isalnum((unsigned char)text[pos - 1]) || text[pos - 1] == '_');
        const char r = pos + len < text.size() ? text[pos + len] : '\0';
        const bool right_ok = !(isalnum((unsigned char)r) || r == '_');
        if (left_ok && right_ok) {
            // a definition: name [dims]... = { ... };  (skip uses of the name that are not followed by '=')
            size_t q = pos + len;
            while (q < text.size() && (isspace((unsigned char)text[q]) || text[q] == '[' || text[q] == ']' || isalnum((unsigned char)text[q]) || text[q] == '_' ||
                                       text[q] == '*' || text[q] == '+' || text[q] == '/'))
                q++;
            if (q < text.size() && text[q] == '=') { pos = q + 1; break; }
        }
        pos += len;
    }
    long seen = 0, stored = 0;
    const char* p = text.c_str() + pos;
    const char* end = text.c_str() + text.size();
    while (p < end && *p != ';' && stored < count) {
        if (p[0] == '/' && p + 1 < end && p[1] == '/') { while (p < end && *p != '\n') p++; continue; }
        if (p[0] == '/' && p + 1 < end && p[1] == '*') { p += 2; while (p + 1 < end && !(p[0] == '*' && p[1] == '/')) p++; p += 2; continue; }
        if (isdigit((unsigned char)*p) || *p == '-' || *p == '+' || *p == '.') {
            char* e = nullptr;
            const float v = strtof(p, &e);
            if (e == p) { p++; continue; }
            if (seen >= skip) out[stored++] = v;
            seen++;
            p = e;
            while (p < end && (*p == 'f' || *p == 'F')) p++;
            continue;
        }
        p++;
    }
    return stored;
}

}  // namespace flexllm

using namespace flexllm;

extern "C" int flexllm_ckpt_read_bin(const char* path, size_t offset_bytes, size_t bytes, void* out_host) {
    FLEXLLM_REQUIRE(path && (out_host || bytes == 0));
    FILE* f = fopen(path, "rb");
    if (!f) return FLEXLLM_EIO;
    int rc = FLEXLLM_OK;
    if (fseek(f, (long)offset_bytes, SEEK_SET) != 0 || fread(out_host, 1, bytes, f) != bytes) rc = FLEXLLM_EIO;
    fclose(f);
    return rc;
}

extern "C" int flexllm_ckpt_read_c_array_f32(const char* path, const char* name, long skip, long count, float* out_host) {
    FLEXLLM_REQUIRE(path && name && out_host && skip >= 0 && count >= 0);
    std::string text;
    if (!slurp(path, &text)) return FLEXLLM_EIO;
    const long got = parse_c_array(text, name, skip, count, out_host);
    if (got < 0) return FLEXLLM_EINVAL;          // no such array in the file
    return got == count ? FLEXLLM_OK : FLEXLLM_EIO;
}

extern "C" int flexllm_ckpt_load_layer(const char* dir, int layer, int hidden, int kv_hidden, int ffn, int heads_q,
                                       const flexllm_ckpt_layer_buffers* b) {
    FLEXLLM_REQUIRE(dir && b && layer >= 0 && hidden > 0 && kv_hidden > 0 && ffn > 0 && heads_q > 0);
    struct Proj { const char* name; int out, in; int8_t* w; float* s; float* sum; };
    const Proj projs[7] = {{"q_proj", hidden, hidden, b->wq, b->sq, b->sumq},       {"k_proj", kv_hidden, hidden, b->wk, b->sk, b->sumk},
                           {"v_proj", kv_hidden, hidden, b->wv, b->sv, b->sumv},    {"o_proj", hidden, hidden, b->wo, b->so, b->sumo},
                           {"gate_proj", ffn, hidden, b->wg, b->sg, b->sumg},       {"up_proj", ffn, hidden, b->wu, b->su, b->sumu},
                           {"down_proj", hidden, ffn, b->wd, b->sd, b->sumd}};
    const std::string d = std::string(dir) + "/";
    char buf[64];
    for (const Proj& p : projs) {
        if (p.w) {
            snprintf(buf, sizeof buf, "%s_L%02d.bin", p.name, layer);
            TRY_RC(flexllm_ckpt_read_bin((d + buf).c_str(), 0, (size_t)p.out * p.in, p.w));
        }
        if (p.s || p.sum) {
            const std::string hdr = d + "w_" + p.name + "_s_sum.h";
            std::string text;
            if (!slurp(hdr, &text)) return FLEXLLM_EIO;
            const std::string ns = std::string("w_") + p.name + "_s", nsum = std::string("w_") + p.name + "_sum";
            if (p.s && parse_c_array(text, ns.c_str(), (long)layer * p.out, p.out, p.s) != p.out) return FLEXLLM_EIO;
            if (p.sum && parse_c_array(text, nsum.c_str(), (long)layer * p.out, p.out, p.sum) != p.out) return FLEXLLM_EIO;
        }
    }
    if (b->gamma0) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "w_rmsnorm.h").c_str(), "RMSNorm_weight", (long)(2 * layer) * hidden, hidden, b->gamma0));
    if (b->gamma1) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "w_rmsnorm.h").c_str(), "RMSNorm_weight", (long)(2 * layer + 1) * hidden, hidden, b->gamma1));
    if (b->a_s) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "A_s.h").c_str(), "A_s", (long)layer * heads_q, heads_q, b->a_s));
    return FLEXLLM_OK;
}

extern "C" int flexllm_ckpt_load_head(const char* dir, int layers, int hidden, int vocab, int table_len, int8_t* lm_w, float* lm_s,
                                      float* lm_sum, float* gamma_final, float* cos_t, float* sin_t, float* embed) {
    FLEXLLM_REQUIRE(dir && layers > 0 && hidden > 0 && vocab > 0 && table_len >= 0);
    const std::string d = std::string(dir) + "/";
    if (lm_w) TRY_RC(flexllm_ckpt_read_bin((d + "lm_head_L00.bin").c_str(), 0, (size_t)vocab * hidden, lm_w));
    if (lm_s) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "w_lm_head_lm_head.h").c_str(), "w_lm_head_lm_head_s", 0, vocab, lm_s));
    if (lm_sum) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "w_lm_head_lm_head.h").c_str(), "w_lm_head_lm_head_sum", 0, vocab, lm_sum));
    if (gamma_final) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "w_rmsnorm.h").c_str(), "RMSNorm_weight", (long)(2 * layers) * hidden, hidden, gamma_final));
    if (cos_t) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "RoPE_sin_cos.h").c_str(), "PE_cos", 0, (long)table_len * 32, cos_t));
    if (sin_t) TRY_RC(flexllm_ckpt_read_c_array_f32((d + "RoPE_sin_cos.h").c_str(), "PE_sin", 0, (long)table_len * 32, sin_t));
    if (embed) TRY_RC(flexllm_ckpt_read_bin((d + "model_embed_tokens_fp32.bin").c_str(), 0, (size_t)vocab * hidden * sizeof(float), embed));
    return FLEXLLM_OK;
}
