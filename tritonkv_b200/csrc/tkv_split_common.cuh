// Pieces shared by the two split-K decode kernels (packed-KV and fp16 control):
// launch parameters, the per-warp online-softmax update and the CTA epilogue that
// merges the warps' partial results and writes either the split partial or the
// normalised output.
#pragma once

#include "tkv_common.cuh"

namespace tkv {

constexpr int kTile = 16;        // tokens per warp tile (one MMA M/K extent)
constexpr int kHeadsPerCta = 8;  // query heads served per CTA (one MMA N extent)

struct DecodeParams {
  const void* q;
  int q_dtype;
  // packed cache (fused kernel)
  const uint8_t* kp;
  const uint8_t* vp;
  const __half* ks;
  const __half* kz;
  const __half* vs;
  const __half* vz;
  // fp16 cache (control kernel)
  const __half* k;
  const __half* v;
  float* acc;
  float* m;
  float* l;
  float* out;
  const int32_t* seq_lens;
  int B, HQ, HKV, S;
  int group;       // HQ / HKV
  int hchunks;     // ceil(group / 8): CTAs per KV head along the head axis
  int num_splits;
  int split_size;  // tokens per split, multiple of 16
  float qk_scale;  // sm_scale * log2(e)
  int partials;    // 1: write (acc, m, l); 0: write normalised out
  int meta_aligned;  // bytes every scale/zero tile start is aligned to: 16, 8, 4, or 0 (2 bytes only)
  int meta_phase;    // with meta_aligned == 0: the scale/zero pointers modulo 4 (0 or 2)
  int wide;          // 1: code tensors are fetched as 128-byte rows (128B TMA swizzle)
};

// Running softmax state of one warp for the two heads (2t, 2t+1) a lane owns.
struct SoftmaxState {
  float m0, m1;  // running maxima (exp2 domain), identical across the 8 lanes sharing t
  float l0, l1;  // per-lane partial sums of p
};

// Scores sc[0..3] = (token g, head 2t), (token g, head 2t+1), (token g+8, head 2t),
// (token g+8, head 2t+1), already multiplied by qk_scale.  Updates the running
// maxima, turns sc into probabilities p = 2^(sc - m) in place and returns whether
// any lane's maximum moved (then alpha0/alpha1 hold the rescale factors that the
// caller must apply to its accumulators).
__device__ __forceinline__ bool softmax_update(SoftmaxState& st, float (&sc)[4], float& alpha0,
                                               float& alpha1) {
  float mx0 = fmaxf(sc[0], sc[2]);
  float mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, off));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, off));
  }
  const float mn0 = fmaxf(st.m0, mx0);
  const float mn1 = fmaxf(st.m1, mx1);
  const bool moved = __any_sync(kFullMask, (mn0 > st.m0) || (mn1 > st.m1));
  if (moved) {
    alpha0 = ex2(st.m0 - mn0);  // first tile: 2^(-inf) = 0
    alpha1 = ex2(st.m1 - mn1);
    st.l0 *= alpha0;
    st.l1 *= alpha1;
    st.m0 = mn0;
    st.m1 = mn1;
  }
  sc[0] = ex2(sc[0] - st.m0);
  sc[1] = ex2(sc[1] - st.m1);
  sc[2] = ex2(sc[2] - st.m0);
  sc[3] = ex2(sc[3] - st.m1);
  st.l0 += sc[0] + sc[2];
  st.l1 += sc[1] + sc[3];
  return moved;
}

// Shared-memory layout of the CTA epilogue: vals[warp][8][D], then m[warp][8], l[warp][8].
template <int D>
__device__ __forceinline__ float* merge_vals(uint8_t* smem, int warp) {
  return reinterpret_cast<float*>(smem) + warp * kHeadsPerCta * D;
}
template <int D>
__device__ __forceinline__ float* merge_ml(uint8_t* smem, int nwarps) {
  return reinterpret_cast<float*>(smem) + nwarps * kHeadsPerCta * D;
}
template <int D>
constexpr int merge_bytes(int nwarps) {
  return nwarps * kHeadsPerCta * (D + 2) * 4;
}

// Each lane publishes its warp's (m, l) for its two heads; lanes with g == 0 write.
// l0/l1 must already be summed over the 8 lanes that share t.
template <int D>
__device__ __forceinline__ void publish_ml(uint8_t* smem, int nwarps, int warp, int lane,
                                           const SoftmaxState& st) {
  float* ml = merge_ml<D>(smem, nwarps);
  if ((lane >> 2) == 0) {
    const int t = lane & 3;
    ml[warp * 8 + 2 * t] = st.m0;
    ml[warp * 8 + 2 * t + 1] = st.m1;
    ml[nwarps * 8 + warp * 8 + 2 * t] = st.l0;
    ml[nwarps * 8 + warp * 8 + 2 * t + 1] = st.l1;
  }
}

// Log-sum-exp merge of the warps' partials, then the global store.
template <int D>
__device__ __forceinline__ void cta_merge_store(const DecodeParams& p, uint8_t* smem, int nwarps,
                                                int b, int hkv, int hc, int split) {
  const float* vals = reinterpret_cast<const float*>(smem);
  const float* ml = merge_ml<D>(smem, nwarps);
  for (int idx = threadIdx.x; idx < kHeadsPerCta * D; idx += blockDim.x) {
    const int h = idx / D, d = idx % D;
    const int hg = hc * kHeadsPerCta + h;
    if (hg >= p.group) continue;
    float M = -INFINITY;
    for (int w = 0; w < nwarps; ++w) M = fmaxf(M, ml[w * 8 + h]);
    float a = 0.f, L = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      const float mw = ml[w * 8 + h];
      const float s = (mw == -INFINITY) ? 0.f : ex2(mw - M);
      a = fmaf(s, vals[(w * kHeadsPerCta + h) * D + d], a);
      L = fmaf(s, ml[nwarps * 8 + w * 8 + h], L);
    }
    const int64_t hq = (int64_t)b * p.HQ + hkv * p.group + hg;
    if (p.partials) {
      const int64_t pi = hq * p.num_splits + split;
      p.acc[pi * D + d] = a;
      if (d == 0) {
        p.m[pi] = M;
        p.l[pi] = L;
      }
    } else {
      p.out[hq * D + d] = (L > 0.f) ? a / L : 0.f;
    }
  }
}

}  // namespace tkv
