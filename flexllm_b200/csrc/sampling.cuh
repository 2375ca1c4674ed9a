// Top-k sampling of the reference's decode graph (Modules/Logits.h:145-279 as instantiated in
// SpinQuant_Llama_32_1B/SpinQuant_Decoding_mem_opt.h:934: inner_block_parallel 1, enable_sub_max),
// one row per call by a group of NT threads. Shared by the stand-alone kernel and the persistent
// decode-step kernel.
//
// The reference splits the vocabulary into `lanes` contiguous slices; every lane keeps an insertion-
// sorted top-k of its slice (sort_top_k, Logits.h:5-31: strict '>', so equal values stay in index
// order); the lanes' lists are merged by inserting rank 0 of every lane, then rank 1, ... into one
// more sorted list; softmax over the k winners (two interleaved partial sums), cumulative
// probabilities, and the first k whose cumulative probability exceeds the host-supplied uniform
// number is the token (else the last). Here a warp owns a lane: each thread keeps the top-k of its
// strided share (same strict '>' insertion in index order), the warp extracts the lane's list by k
// rounds of "largest value, lowest index first", and one thread replays the reference's merge and
// sampling verbatim, so ties resolve exactly as they do there.
#pragma once
#include <math.h>

#include "common.cuh"

namespace flexllm {

constexpr int SAMPLE_KMAX = 8;       // largest top_k (the accelerator configs use 5)
constexpr int SAMPLE_LMAX = 64;      // largest lane count

struct SampleSmem {
    float lane_val[SAMPLE_LMAX][SAMPLE_KMAX];
    int lane_idx[SAMPLE_LMAX][SAMPLE_KMAX];
};

// Returns the sampled index to thread 0 of the group (other threads get -1). top_idx / top_val (optional,
// k entries) receive the merged list. `bar`: named barrier of the group's NT threads.
template <int NT>
__device__ __forceinline__ int topk_sample_row(const float* __restrict__ l, const long V, const int lanes, const int top_k,
                                               const float rnd, SampleSmem& sm, const int tid, const int bar,
                                               int32_t* top_idx, float* top_val) {
    const int w = tid >> 5, lane = tid & 31;
    const long seg = V / lanes;
    for (int i = w; i < lanes; i += NT / 32) {
        // this thread's share of slice i: elements lane, lane + 32, ... in increasing index order
        float val[SAMPLE_KMAX];
        int idx[SAMPLE_KMAX];
#pragma unroll
        for (int k = 0; k < SAMPLE_KMAX; k++) { val[k] = -1e32f; idx[k] = -1; }
        const float* ls = l + (long)i * seg;
        float thr = -1e32f;                      // value at rank top_k - 1: anything not above it cannot enter
        for (long t = lane; t < seg; t += 32) {
            const float v = __ldcg(ls + t);
            if (v > thr) {
                // sort_top_k: the first rank whose value v exceeds takes v, the ranks below shift down
                int pos = top_k;
#pragma unroll
                for (int k = SAMPLE_KMAX - 1; k >= 0; k--)
                    if (k < top_k && v > val[k]) pos = k;
#pragma unroll
                for (int k = SAMPLE_KMAX - 1; k >= 1; k--) {
                    if (k < top_k) {
                        if (k > pos) { val[k] = val[k - 1]; idx[k] = idx[k - 1]; }
                        else if (k == pos) { val[k] = v; idx[k] = (int)(i * seg + t); }
                    }
                }
                if (pos == 0) { val[0] = v; idx[0] = (int)(i * seg + t); }
                thr = val[0];
#pragma unroll
                for (int k = 1; k < SAMPLE_KMAX; k++)
                    if (k < top_k) thr = val[k];
            }
        }
        // the lane's list: k rounds, each takes the best head of the 32 threads (value, then lower index)
        for (int r = 0; r < top_k; r++) {
            float bv = val[0];
            int bi = idx[0], owner = lane;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                const int oo = __shfl_xor_sync(0xffffffffu, owner, o);
                // a real index beats the empty marker (-1) at equal value; among real ones the lower index wins
                const bool better = ov > bv || (ov == bv && (oi >= 0 ? (bi < 0 || oi < bi) : (bi < 0 && oo < owner)));
                if (better) { bv = ov; bi = oi; owner = oo; }
            }
            if (lane == 0) { sm.lane_val[i][r] = bv; sm.lane_idx[i][r] = bi; }
            if (lane == owner) {
#pragma unroll
                for (int k = 0; k < SAMPLE_KMAX - 1; k++) { val[k] = val[k + 1]; idx[k] = idx[k + 1]; }
                val[SAMPLE_KMAX - 1] = -1e32f; idx[SAMPLE_KMAX - 1] = -1;
            }
        }
    }
    named_sync_id<NT>(bar);
    int sampled = -1;
    if (tid == 0) {
        float fval[SAMPLE_KMAX], prob[SAMPLE_KMAX];
        int fid[SAMPLE_KMAX];
        for (int k = 0; k < top_k; k++) { fid[k] = -1; fval[k] = -1e32f; }
        for (int K = 0; K < top_k; K++)
            for (int i = 0; i < lanes; i++) {
                const float v = sm.lane_val[i][K];
                const int vi = sm.lane_idx[i][K];
                int pos = top_k;
                for (int k = 0; k < top_k; k++)
                    if (v > fval[k] && pos == top_k) pos = k;
                for (int k = top_k - 1; k >= 0; k--) {
                    if (k > pos) { fid[k] = fid[k - 1]; fval[k] = fval[k - 1]; }
                    else if (k == pos) { fid[k] = vi; fval[k] = v; }
                }
            }
        float part0 = 0.0f, part1 = 0.0f;
        for (int k = 0; k < top_k; k++) {
            prob[k] = ref_expf(fval[k] - fval[0]);
            if (k & 1) part1 += prob[k]; else part0 += prob[k];
        }
        const float sum = part0 + part1;
        int sel = top_k - 1;
        float cdf = 0.0f;
        for (int k = 0; k < top_k; k++) {
            const float p = prob[k] / sum;
            cdf = k == 0 ? p : p + cdf;
            if (rnd < cdf && sel == top_k - 1) sel = k;
        }
        sampled = fid[sel];
        for (int k = 0; k < top_k; k++) {
            if (top_idx) top_idx[k] = fid[k];
            if (top_val) top_val[k] = fval[k];
        }
    }
    return sampled;
}

}  // namespace flexllm
