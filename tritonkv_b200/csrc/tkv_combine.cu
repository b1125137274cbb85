// Log-sum-exp merge of split-K partials (sm_100a).
//
// Replaces _combine_splits of the reference (kernels/fused_decode_attn.py:355-395):
//     out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),   M = max_s m_s
// One warp per (batch, query head).  The global maximum is found first (lanes
// stride over the splits, warp-shuffle max), then every lane accumulates its
// float4 slice of D over the splits; splits with m = -inf (empty) weigh zero.
// With out_m/out_l given, the merged partial is written unnormalised together
// with (M, L): the wire format of a cross-GPU history split.
#include "tkv_common.cuh"

namespace tkv {

constexpr int kCombineWarps = 4;

__global__ void __launch_bounds__(kCombineWarps * 32)
    combine_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                   const float* __restrict__ l, float* __restrict__ out, float* __restrict__ out_m,
                   float* __restrict__ out_l, int rows, int NS, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kCombineWarps + warp;  // b*HQ + h
  if (row >= rows) return;
  const float* mrow = m + (int64_t)row * NS;
  const float* lrow = l + (int64_t)row * NS;
  const float* arow = acc + (int64_t)row * NS * D;

  float M = -INFINITY;
  for (int s = lane; s < NS; s += 32) M = fmaxf(M, mrow[s]);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(kFullMask, M, off));

  const int nvec = D >> 2;
  float L = 0.f;
  for (int v0 = 0; v0 < nvec; v0 += 32) {
    const int v = v0 + lane;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    float Lloc = 0.f;
    if (v < nvec) {
#pragma unroll 4
      for (int s = 0; s < NS; ++s) {
        const float ms = __ldg(mrow + s);
        const float w = (ms == -INFINITY) ? 0.f : ex2(ms - M);
        const float4 x = __ldg(reinterpret_cast<const float4*>(arow + (int64_t)s * D) + v);
        a.x = fmaf(w, x.x, a.x);
        a.y = fmaf(w, x.y, a.y);
        a.z = fmaf(w, x.z, a.z);
        a.w = fmaf(w, x.w, a.w);
        Lloc = fmaf(w, __ldg(lrow + s), Lloc);
      }
      L = Lloc;
      if (out_m == nullptr) {
        const float inv = Lloc > 0.f ? 1.f / Lloc : 0.f;
        a.x *= inv;
        a.y *= inv;
        a.z *= inv;
        a.w *= inv;
      }
      reinterpret_cast<float4*>(out + (int64_t)row * D)[v] = a;
    }
  }
  if (out_m != nullptr && lane == 0) {
    out_m[row] = M;
    out_l[row] = L;
  }
}

}  // namespace tkv

extern "C" int tkv_combine(const float* acc, const float* m, const float* l, float* out,
                           float* out_m, float* out_l, int B, int HQ, int NS, int D, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(acc && m && l && out, TKV_ERR_INVALID, "combine: null pointer");
  TKV_REQUIRE((out_m == nullptr) == (out_l == nullptr), TKV_ERR_INVALID,
              "combine: out_m and out_l must be given together");
  TKV_REQUIRE(B > 0 && HQ > 0 && NS > 0 && D > 0 && D % 4 == 0, TKV_ERR_INVALID,
              "combine: bad sizes B=%d HQ=%d NS=%d D=%d", B, HQ, NS, D);
  TKV_REQUIRE(aligned16(acc) && aligned16(out), TKV_ERR_ALIGN,
              "combine: acc and out must be 16-byte aligned");
  const int64_t rows = (int64_t)B * HQ;
  TKV_REQUIRE(rows <= (1LL << 30), TKV_ERR_INVALID, "combine: too many rows");
  const int blocks = (int)((rows + kCombineWarps - 1) / kCombineWarps);
  combine_kernel<<<blocks, kCombineWarps * 32, 0, (cudaStream_t)stream>>>(acc, m, l, out, out_m,
                                                                        out_l, (int)rows, NS, D);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}
