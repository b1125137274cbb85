// fp16 control: split-K decode attention on an unquantised f16 cache (sm_100a).
//
// Replaces _fp16_decode_attn_split of the reference (kernels/fp16_decode_attn.py:47-135).
// Same CTA/warp decomposition, ring, online softmax, GQA grouping, partial format and
// epilogue as the packed-cache kernel; only the operand fetch differs: K and V tiles
// are f16 rows, read with ldmatrix (K as the A operand of S^T = K Q^T, V with .trans
// as the A operand of O^T = V^T P^T).
#include "tkv_split_common.cuh"

namespace tkv {

template <int D>
struct Fp16Cfg {
  static constexpr int ROW = 2 * D;           // bytes per token row
  static constexpr int NCHR = ROW / 16;       // 16-byte chunks per row (>= 8)
  static constexpr int NCH = D / 16;          // 16-dim MMA chunks
  static constexpr int TILE_BYTES = kTile * ROW;
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static_assert(NCHR >= 8, "head_dim must be at least 64");
};

template <int D, int STAGES>
__global__ void __launch_bounds__(128, 2) fp16_split_kernel(const DecodeParams p) {
  using C = Fp16Cfg<D>;
  constexpr int NCH = C::NCH, ROW = C::ROW, NCHR = C::NCHR;

  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x;
  const int hkv = blockIdx.y / p.hchunks, hc = blockIdx.y % p.hchunks;
  const int b = blockIdx.z;

  const int S_b = p.seq_lens ? min(max(p.seq_lens[b], 0), p.S) : p.S;
  const int lo = split * p.split_size;
  const int hi = min(lo + p.split_size, S_b);
  const int ntiles = hi > lo ? (hi - lo + kTile - 1) / kTile : 0;
  const int my_tiles = ntiles > warp ? (ntiles - warp + nwarps - 1) / nwarps : 0;
  const int64_t row0 = ((int64_t)b * p.HKV + hkv) * p.S;

  // query fragments: B operand, k-slots (2t,2t+1) <-> dims 16c+2t, 16c+2t+1 and
  // (2t+8, 2t+9) <-> dims 16c+8+2t, 16c+9+2t, column g = head g.
  const int head = hc * kHeadsPerCta + g;
  const bool head_ok = head < p.group;
  const int64_t qoff = ((int64_t)b * p.HQ + (int64_t)hkv * p.group + head) * D;
  uint32_t qf[NCH][2];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    __half x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = 16 * ch + 2 * t + (i & 1) + (i >> 1) * 8;
      x[i] = head_ok ? load_q_half(p.q, p.q_dtype, qoff + d) : __float2half(0.f);
    }
    qf[ch][0] = pack_half2(x[0], x[1]);
    qf[ch][1] = pack_half2(x[2], x[3]);
  }

  uint8_t* ring = smem + (size_t)warp * STAGES * C::STAGE_BYTES;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint8_t* k_row = reinterpret_cast<const uint8_t*>(p.k) + row0 * ROW;
  const uint8_t* v_row = reinterpret_cast<const uint8_t*>(p.v) + row0 * ROW;

  auto issue = [&](int j) {
    const int slot = j % STAGES;
    const int tok0 = lo + (warp + j * nwarps) * kTile;
    const int nvalid = min(kTile, hi - tok0);
    const uint32_t st = ring_u32 + slot * C::STAGE_BYTES;
    constexpr int NCC = kTile * NCHR;
#pragma unroll
    for (int i0 = 0; i0 < NCC; i0 += 32) {
      const int i = i0 + lane;
      const int r = i / NCHR, chunk = i % NCHR;
      const uint32_t dst = r * ROW + ((chunk ^ (r & 7)) << 4);
      const bool ok = r < nvalid;
      const int64_t src = (int64_t)tok0 * ROW + i * 16;
      cp_async16(st + dst, ok ? k_row + src : (const uint8_t*)p.k, ok ? 16 : 0);
      cp_async16(st + C::TILE_BYTES + dst, ok ? v_row + src : (const uint8_t*)p.v, ok ? 16 : 0);
    }
  };

  SoftmaxState sm_state{-INFINITY, -INFINITY, 0.f, 0.f};
  float acc[NCH][4];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[ch][i] = 0.f;

  // ldmatrix addressing.  K (A operand, row-major tokens x dims): matrices
  // (tok 0-7, chunk 2c), (tok 8-15, chunk 2c), (tok 0-7, chunk 2c+1), (tok 8-15, chunk 2c+1).
  const int k_r = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int k_c = lane >> 4;
  // V (A operand of O^T, via .trans): matrices (tok 0-7, chunk 2i), (tok 0-7, chunk 2i+1),
  // (tok 8-15, chunk 2i), (tok 8-15, chunk 2i+1).
  const int v_r = (lane & 7) + (lane >> 4) * 8;
  const int v_c = (lane >> 3) & 1;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < my_tiles) issue(s);
    cp_async_commit();
  }

  for (int j = 0; j < my_tiles; ++j) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (j + STAGES - 1 < my_tiles) issue(j + STAGES - 1);
    cp_async_commit();

    const int slot = j % STAGES;
    const int tok0 = lo + (warp + j * nwarps) * kTile;
    const int nvalid = hi - tok0;
    const uint32_t kt = ring_u32 + slot * C::STAGE_BYTES;
    const uint32_t vt = kt + C::TILE_BYTES;

    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      uint32_t r[4];
      ldmatrix_x4(r, kt + k_r * ROW + ((((2 * ch + k_c)) ^ (k_r & 7)) << 4));
      mma16816(sc, r[0], r[1], r[2], r[3], qf[ch][0], qf[ch][1]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i] *= p.qk_scale;
    if (nvalid < kTile) {
      if (g >= nvalid) sc[0] = sc[1] = -INFINITY;
      if (g + 8 >= nvalid) sc[2] = sc[3] = -INFINITY;
    }

    float alpha0, alpha1;
    if (softmax_update(sm_state, sc, alpha0, alpha1)) {
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        acc[ch][0] *= alpha0;
        acc[ch][1] *= alpha1;
        acc[ch][2] *= alpha0;
        acc[ch][3] *= alpha1;
      }
    }

    const uint32_t pb0 = movmatrix_trans(pack_half2(sc[0], sc[1]));
    const uint32_t pb1 = movmatrix_trans(pack_half2(sc[2], sc[3]));
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      uint32_t r[4];
      ldmatrix_x4_trans(r, vt + v_r * ROW + (((2 * ch + v_c) ^ (v_r & 7)) << 4));
      mma16816(acc[ch], r[0], r[1], r[2], r[3], pb0, pb1);
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    sm_state.l0 += __shfl_xor_sync(kFullMask, sm_state.l0, off);
    sm_state.l1 += __shfl_xor_sync(kFullMask, sm_state.l1, off);
  }
  __syncthreads();
  float* vals = merge_vals<D>(smem, warp);
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    // rows g / g+8 of output tile ch are dims 16ch+g / 16ch+8+g; columns heads 2t, 2t+1
    vals[(2 * t) * D + 16 * ch + g] = acc[ch][0];
    vals[(2 * t + 1) * D + 16 * ch + g] = acc[ch][1];
    vals[(2 * t) * D + 16 * ch + 8 + g] = acc[ch][2];
    vals[(2 * t + 1) * D + 16 * ch + 8 + g] = acc[ch][3];
  }
  publish_ml<D>(smem, nwarps, warp, lane, sm_state);
  __syncthreads();
  cta_merge_store<D>(p, smem, nwarps, b, hkv, hc, split);
}

constexpr int kFp16Warps = 4;

template <int D>
struct Fp16Launch {
  static constexpr int STAGES = (D >= 128) ? 3 : 4;
  static int smem_bytes() {
    const int ring = kFp16Warps * STAGES * Fp16Cfg<D>::STAGE_BYTES;
    const int merge = merge_bytes<D>(kFp16Warps);
    return ring > merge ? ring : merge;
  }
  static const void* fn() { return reinterpret_cast<const void*>(&fp16_split_kernel<D, STAGES>); }
  static int prepare() {
    static bool done[64] = {};
    int dev = 0;
    TKV_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && done[dev]) return TKV_OK;
    TKV_CUDA(cudaFuncSetAttribute(fn(), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes()));
    if (dev < 64) done[dev] = true;
    return TKV_OK;
  }
  static int launch(const DecodeParams& p, cudaStream_t stream) {
    int rc = prepare();
    if (rc != TKV_OK) return rc;
    dim3 grid(p.num_splits, p.HKV * p.hchunks, p.B);
    fp16_split_kernel<D, STAGES><<<grid, kFp16Warps * 32, smem_bytes(), stream>>>(p);
    TKV_CUDA(cudaGetLastError());
    return TKV_OK;
  }
  static int attrs(int* regs, int* smem, int* local, int* ctas) {
    int rc = prepare();
    if (rc != TKV_OK) return rc;
    cudaFuncAttributes a;
    TKV_CUDA(cudaFuncGetAttributes(&a, fn()));
    if (regs) *regs = a.numRegs;
    if (smem) *smem = (int)a.sharedSizeBytes + smem_bytes();
    if (local) *local = (int)a.localSizeBytes;
    if (ctas) {
      int n = 0;
      TKV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn(), kFp16Warps * 32,
                                                             smem_bytes()));
      *ctas = n;
    }
    return TKV_OK;
  }
};

int fp16_attrs(int D, int* regs, int* smem, int* local, int* ctas) {
  if (D == 128) return Fp16Launch<128>::attrs(regs, smem, local, ctas);
  if (D == 64) return Fp16Launch<64>::attrs(regs, smem, local, ctas);
  set_error("fp16 decode: unsupported head_dim=%d (built: 64, 128)", D);
  return TKV_ERR_UNSUPPORTED;
}

}  // namespace tkv

extern "C" int tkv_fp16_decode(const void* q, int q_dtype, const void* k, const void* v, float* acc,
                               float* m, float* l, float* out, int B, int HQ, int HKV, int S, int D,
                               float sm_scale, int num_splits, int split_size,
                               const int32_t* seq_lens, int flags, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(q && k && v, TKV_ERR_INVALID, "fp16 decode: null input pointer");
  TKV_REQUIRE(B > 0 && HQ > 0 && HKV > 0 && S > 0, TKV_ERR_INVALID,
              "fp16 decode: B, HQ, HKV, S must be positive (got %d, %d, %d, %d)", B, HQ, HKV, S);
  TKV_REQUIRE(B <= 65535, TKV_ERR_INVALID, "fp16 decode: batch %d exceeds 65535", B);
  TKV_REQUIRE(HQ % HKV == 0, TKV_ERR_INVALID, "HQ=%d must be a multiple of HKV=%d", HQ, HKV);
  TKV_REQUIRE(q_dtype >= 0 && q_dtype <= 2, TKV_ERR_INVALID, "fp16 decode: bad q dtype %d", q_dtype);
  TKV_REQUIRE(num_splits >= 1 && split_size >= 16 && split_size % 16 == 0, TKV_ERR_INVALID,
              "fp16 decode: split_size=%d must be a positive multiple of 16, num_splits=%d >= 1",
              split_size, num_splits);
  TKV_REQUIRE((int64_t)num_splits * split_size >= S, TKV_ERR_INVALID,
              "fp16 decode: %d splits of %d tokens do not cover S=%d", num_splits, split_size, S);
  const bool partials = num_splits > 1 || (flags & TKV_FLAG_PARTIALS_ONLY);
  TKV_REQUIRE(!partials || (acc && m && l), TKV_ERR_INVALID,
              "fp16 decode: partial buffers (acc, m, l) required");
  TKV_REQUIRE(partials || out, TKV_ERR_INVALID, "fp16 decode: out required");
  TKV_REQUIRE(aligned16(k) && aligned16(v), TKV_ERR_ALIGN,
              "fp16 decode: k and v pointers must be 16-byte aligned");
  DecodeParams p{};
  p.q = q;
  p.q_dtype = q_dtype;
  p.k = (const __half*)k;
  p.v = (const __half*)v;
  p.acc = acc;
  p.m = m;
  p.l = l;
  p.out = out;
  p.seq_lens = seq_lens;
  p.B = B;
  p.HQ = HQ;
  p.HKV = HKV;
  p.S = S;
  p.group = HQ / HKV;
  p.hchunks = (p.group + kHeadsPerCta - 1) / kHeadsPerCta;
  p.num_splits = num_splits;
  p.split_size = split_size;
  p.qk_scale = sm_scale * kLog2e;
  p.partials = partials ? 1 : 0;
  TKV_REQUIRE((int64_t)HKV * p.hchunks <= 65535, TKV_ERR_INVALID, "fp16 decode: too many heads");
  if (D == 128) return Fp16Launch<128>::launch(p, (cudaStream_t)stream);
  if (D == 64) return Fp16Launch<64>::launch(p, (cudaStream_t)stream);
  set_error("fp16 decode: unsupported head_dim=%d (built: 64, 128)", D);
  return TKV_ERR_UNSUPPORTED;
}
