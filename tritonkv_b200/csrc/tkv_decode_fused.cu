// Fused split-K decode attention on a packed 2/4-bit KV cache (sm_100a).
//
// Replaces _fused_decode_attn_split of the reference (kernels/fused_decode_attn.py:155-353).
//
// One CTA serves one (batch, KV head, history split) and up to 8 query heads of the
// GQA group.  Inside the CTA every warp is an independent stream: it owns a private
// ring of shared-memory stages filled with 16-byte cp.async copies, walks its own
// 16-token tiles of the split, and keeps a private online-softmax state; the warps'
// results are merged once, in the epilogue.  No CTA-wide barrier sits in the loop.
//
// Arithmetic.  The packed bytes are never expanded to dequantised values.  With
// code c, group scale s and group zero z, a cache value is c*s + z, so
//     q.k = sum_g s_g * (sum_{d in g} q_d c_d)  +  sum_g z_g * (sum_{d in g} q_d)
//     sum_n p_n v_n[d] = sum_n (p_n s_{n,g(d)}) c_n[d]  +  sum_n p_n z_{n,g(d)}
// The inner sums are tensor-core MMAs (m16n8k16, f16 in, f32 accumulate) whose
// A operand is the raw code field, isolated from the packed word by ONE bitwise AND:
// a 2- or 4-bit field inside the mantissa of an f16 is the subnormal (or scaled)
// number c * 2^(pos-24), exact, and the power of two is folded into the f32 scale
// afterwards.  The zero-point terms are one extra MMA each per tile.  Per packed
// 32-bit word (8 or 16 codes) the integer work is one shift and P*2 ANDs.
//
// Fragment mapping (g = lane/4, t = lane%4).  Scores use S^T = K Q^T with the 16
// tokens of a tile as MMA rows and the 8 heads as columns; the output uses
// O^T = V^T P^T with 16 head-dims as rows.  ldmatrix delivers for K the 4 bytes
// [16b+4t, 16b+4t+4) of tokens g / g+8, and with .trans for V the 2 bytes
// [16b+2g, 16b+2g+2) of token pairs (2t, 2t+1) / (2t+8, 2t+9) -- already in the
// layout of an A fragment once masked.  Chunk ch = slice*NBLK + b covers head dims
// [16ch, 16ch+16) because of the split-P layout (byte j, bit slice p -> dim j + p*DP).
#include "tkv_split_common.cuh"

namespace tkv {

template <int NBITS, int D, int GS>
struct FusedCfg {
  static constexpr int P = 8 / NBITS;          // codes per byte = bit slices
  static constexpr int DP = D / P;             // packed bytes per token
  static constexpr int NBLK = DP / 16;         // 16-byte column blocks per token row
  static constexpr int NCH = D / 16;           // 16-dim chunks
  static constexpr int NG = D / GS;            // quantisation groups per token
  static constexpr int ACC_DIMS = (GS < DP) ? GS : DP;  // dims sharing one score accumulator
  static constexpr int NACC = D / ACC_DIMS;
  static constexpr int CODE_BYTES = kTile * DP;
  static constexpr int META_BYTES = kTile * NG * 2;
  static constexpr int STAGE_BYTES = 2 * CODE_BYTES + 4 * META_BYTES;
  static constexpr uint32_t MASK0 = ((1u << NBITS) - 1u) * 0x00010001u;
  static constexpr int SWZ_SHIFT = (NBLK == 4) ? 1 : 2;
  static_assert(NBLK == 1 || NBLK == 2 || NBLK == 4, "packed row must be 16, 32 or 64 bytes");
  static_assert(GS >= 16 && NG >= 1 && NG <= 8, "group size must be 16..D with at most 8 groups");
};

template <int NG>
__device__ __forceinline__ void load_meta_row(const __half* p, __half (&out)[NG]) {
  if constexpr (NG == 8) {
    *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(p);
  } else if constexpr (NG == 4) {
    *reinterpret_cast<uint2*>(out) = *reinterpret_cast<const uint2*>(p);
  } else if constexpr (NG == 2) {
    *reinterpret_cast<uint32_t*>(out) = *reinterpret_cast<const uint32_t*>(p);
  } else {
    out[0] = p[0];
  }
}

template <int NBITS, int D, int GS, int STAGES>
__global__ void __launch_bounds__(128, 3) fused_split_kernel(const DecodeParams p) {
  using C = FusedCfg<NBITS, D, GS>;
  constexpr int P = C::P, DP = C::DP, NBLK = C::NBLK, NCH = C::NCH, NG = C::NG;
  constexpr int NACC = C::NACC, ACC_DIMS = C::ACC_DIMS;

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

  // ---- query fragments (B operand of the score MMA) and per-group query sums ----
  const int head = hc * kHeadsPerCta + g;
  const bool head_ok = head < p.group;
  const int64_t qoff = ((int64_t)b * p.HQ + (int64_t)hkv * p.group + head) * D;
  uint32_t qf[NCH][2];
  float gsum[NG];
#pragma unroll
  for (int i = 0; i < NG; ++i) gsum[i] = 0.f;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    __half x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      x[i] = head_ok ? load_q_half(p.q, p.q_dtype, qoff + 16 * ch + 4 * t + i) : __float2half(0.f);
    qf[ch][0] = pack_half2(x[0], x[2]);  // k-slots 2t, 2t+1   <-> dims 16ch+4t, 16ch+4t+2
    qf[ch][1] = pack_half2(x[1], x[3]);  // k-slots 2t+8, 2t+9 <-> dims 16ch+4t+1, 16ch+4t+3
    gsum[(16 * ch) / GS] += (__half2float(x[0]) + __half2float(x[1])) +
                            (__half2float(x[2]) + __half2float(x[3]));
  }
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    gsum[i] += __shfl_xor_sync(kFullMask, gsum[i], 1);
    gsum[i] += __shfl_xor_sync(kFullMask, gsum[i], 2);
  }
  // B operand of the K zero-point MMA: k-slots (2t, 2t+1) carry the f16 hi/lo split of
  // the query sum of group t, k-slots (2t+8, 2t+9) that of group t+4.
  uint32_t qz0 = 0, qz1 = 0;
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const __half hi16 = __float2half_rn(gsum[i]);
    const __half lo16 = __float2half_rn(gsum[i] - __half2float(hi16));
    const uint32_t v = pack_half2(hi16, lo16);
    if (i == t) qz0 = v;
    if (i == t + 4) qz1 = v;
  }

  // ---- per-warp ring ----
  uint8_t* ring = smem + (size_t)warp * STAGES * C::STAGE_BYTES;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint8_t* kp_row = p.kp + row0 * DP;
  const uint8_t* vp_row = p.vp + row0 * DP;
  const __half* meta_row[4] = {p.ks + row0 * NG, p.kz + row0 * NG, p.vs + row0 * NG,
                               p.vz + row0 * NG};

  auto issue = [&](int j) {
    const int slot = j % STAGES;
    const int tok0 = lo + (warp + j * nwarps) * kTile;
    const int nvalid = min(kTile, hi - tok0);
    const uint32_t st = ring_u32 + slot * C::STAGE_BYTES;
    constexpr int NCC = kTile * NBLK;  // 16-byte chunks per code tile
#pragma unroll
    for (int i0 = 0; i0 < NCC; i0 += 32) {
      const int i = i0 + lane;
      if (NCC >= 32 || i < NCC) {
        const int r = i / NBLK, blk = i % NBLK;
        const int swz = (NBLK > 1) ? ((r >> C::SWZ_SHIFT) & (NBLK - 1)) : 0;
        const uint32_t dst = r * DP + ((blk ^ swz) << 4);
        const bool ok = r < nvalid;
        const int64_t src = (int64_t)tok0 * DP + i * 16;
        cp_async16(st + dst, ok ? kp_row + src : p.kp, ok ? 16 : 0);
        cp_async16(st + C::CODE_BYTES + dst, ok ? vp_row + src : p.vp, ok ? 16 : 0);
      }
    }
    const uint32_t mst = st + 2 * C::CODE_BYTES;
    if (p.meta_aligned) {
      constexpr int CPA = C::META_BYTES / 16;   // chunks per metadata array
      constexpr int TOK_BYTES = NG * 2;         // metadata bytes per token
#pragma unroll
      for (int i0 = 0; i0 < 4 * CPA; i0 += 32) {
        const int i = i0 + lane;
        if (4 * CPA >= 32 || i < 4 * CPA) {
          const int arr = i / CPA, c = i % CPA;
          const int valid_bytes = max(0, min(16, nvalid * TOK_BYTES - c * 16));
          const uint8_t* src = reinterpret_cast<const uint8_t*>(meta_row[arr]) +
                               (int64_t)tok0 * TOK_BYTES + c * 16;
          cp_async16(mst + i * 16, valid_bytes > 0 ? src : (const uint8_t*)p.ks, valid_bytes);
        }
      }
    } else {
      // Rows that do not start on 16-byte boundaries (odd history lengths): plain loads.
      __half* dstm = reinterpret_cast<__half*>(ring + slot * C::STAGE_BYTES + 2 * C::CODE_BYTES);
#pragma unroll
      for (int arr = 0; arr < 4; ++arr)
        for (int i = lane; i < kTile * NG; i += 32) {
          const int tok = i / NG;
          dstm[arr * kTile * NG + i] =
              tok < nvalid ? meta_row[arr][(int64_t)tok0 * NG + i] : __float2half(0.f);
        }
    }
  };

  // ---- running state ----
  SoftmaxState sm_state{-INFINITY, -INFINITY, 0.f, 0.f};
  float acc[NCH][4];
  float zacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[ch][i] = 0.f;

  const int lm_r = (lane & 7) + ((lane >> 3) & 1) * 8;  // token row this lane addresses
  const int lm_b = lane >> 4;                           // column-block offset (x4 only)
  const int lm_swz = (NBLK > 1) ? ((lm_r >> C::SWZ_SHIFT) & (NBLK - 1)) : 0;
  const uint32_t lm_row_off = lm_r * DP;

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
    const int nvalid = hi - tok0;  // >= 1; may exceed 16
    const uint32_t kc = ring_u32 + slot * C::STAGE_BYTES;
    const uint32_t vc = kc + C::CODE_BYTES;
    const __half* ks_s = reinterpret_cast<const __half*>(ring + slot * C::STAGE_BYTES + 2 * C::CODE_BYTES);
    const __half* kz_s = ks_s + kTile * NG;
    const __half* vs_s = kz_s + kTile * NG;
    const __half* vz_s = vs_s + kTile * NG;

    // ================= scores: S^T = K Q^T, one accumulator per (slice, group) ========
    float c[NACC][4];
#pragma unroll
    for (int a = 0; a < NACC; ++a)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[a][i] = 0.f;
#pragma unroll
    for (int bb = 0; bb < NBLK; bb += 2) {
      uint32_t r[4];
      if constexpr (NBLK >= 2) {
        ldmatrix_x4(r, kc + lm_row_off + (((bb + lm_b) ^ lm_swz) << 4));
      } else {
        ldmatrix_x2(r[0], r[1], kc + lm_row_off);
        r[2] = r[3] = 0;
      }
#pragma unroll
      for (int jj = 0; jj < (NBLK >= 2 ? 2 : 1); ++jj) {
        const int blk = bb + jj;
        const uint32_t xl = r[2 * jj], xh = r[2 * jj + 1];
        const uint32_t xl8 = xl >> 8, xh8 = xh >> 8;
#pragma unroll
        for (int pp = 0; pp < P; ++pp) {
          constexpr uint32_t M0 = C::MASK0;
          const uint32_t mask = M0 << (NBITS * pp);
          const int ch = pp * NBLK + blk;
          mma16816(c[(16 * ch) / ACC_DIMS], xl & mask, xh & mask, xl8 & mask, xh8 & mask,
                   qf[ch][0], qf[ch][1]);
        }
      }
    }
    // zero-point term: sum_g z[token][g] * qsum[g][head]
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    {
      uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
      if (t < NG) {
        const __half z0 = kz_s[g * NG + t], z1 = kz_s[(g + 8) * NG + t];
        a0 = pack_half2(z0, z0);
        a1 = pack_half2(z1, z1);
      }
      if (NG == 8) {
        const __half z0 = kz_s[g * NG + (t + 4) % NG], z1 = kz_s[(g + 8) * NG + (t + 4) % NG];
        a2 = pack_half2(z0, z0);
        a3 = pack_half2(z1, z1);
      }
      mma16816(sc, a0, a1, a2, a3, qz0, qz1);
    }
    // scale term
    {
      __half s_lo[NG], s_hi[NG];
      load_meta_row<NG>(ks_s + g * NG, s_lo);
      load_meta_row<NG>(ks_s + (g + 8) * NG, s_hi);
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        const int grp = (a * ACC_DIMS) / GS;
        const int slice = (a * ACC_DIMS) / DP;
        const float e = pow2i(24 - NBITS * slice);
        const float f_lo = __half2float(s_lo[grp]) * e;
        const float f_hi = __half2float(s_hi[grp]) * e;
        sc[0] = fmaf(c[a][0], f_lo, sc[0]);
        sc[1] = fmaf(c[a][1], f_lo, sc[1]);
        sc[2] = fmaf(c[a][2], f_hi, sc[2]);
        sc[3] = fmaf(c[a][3], f_hi, sc[3]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i] *= p.qk_scale;
    if (nvalid < kTile) {
      if (g >= nvalid) sc[0] = sc[1] = -INFINITY;
      if (g + 8 >= nvalid) sc[2] = sc[3] = -INFINITY;
    }

    // ================= online softmax ===============================================
    float alpha0, alpha1;
    if (softmax_update(sm_state, sc, alpha0, alpha1)) {
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        acc[ch][0] *= alpha0;
        acc[ch][1] *= alpha1;
        acc[ch][2] *= alpha0;
        acc[ch][3] *= alpha1;
      }
      zacc[0] *= alpha0;
      zacc[1] *= alpha1;
    }

    // ================= output: O^T += V^T P^T ========================================
    const uint32_t ph_lo = pack_half2(sc[0], sc[1]);  // token g,   heads 2t, 2t+1
    const uint32_t ph_hi = pack_half2(sc[2], sc[3]);  // token g+8
    {
      // zero-point term: rows = groups, k = tokens; B = unscaled P^T
      const uint32_t pz0 = movmatrix_trans(ph_lo);
      const uint32_t pz1 = movmatrix_trans(ph_hi);
      uint32_t a0 = 0, a2 = 0;
      if (g < NG) {
        a0 = pack_half2(vz_s[(2 * t) * NG + g], vz_s[(2 * t + 1) * NG + g]);
        a2 = pack_half2(vz_s[(2 * t + 8) * NG + g], vz_s[(2 * t + 9) * NG + g]);
      }
      mma16816(zacc, a0, 0u, a2, 0u, pz0, pz1);
    }
    uint32_t pb[NG][2];
    {
      __half s_lo[NG], s_hi[NG];
      load_meta_row<NG>(vs_s + g * NG, s_lo);
      load_meta_row<NG>(vs_s + (g + 8) * NG, s_hi);
#pragma unroll
      for (int grp = 0; grp < NG; ++grp) {
        pb[grp][0] = movmatrix_trans(hmul2_u32(ph_lo, pack_half2(s_lo[grp], s_lo[grp])));
        pb[grp][1] = movmatrix_trans(hmul2_u32(ph_hi, pack_half2(s_hi[grp], s_hi[grp])));
      }
    }
#pragma unroll
    for (int bb = 0; bb < NBLK; bb += 2) {
      uint32_t r[4];
      if constexpr (NBLK >= 2) {
        ldmatrix_x4_trans(r, vc + lm_row_off + (((bb + lm_b) ^ lm_swz) << 4));
      } else {
        ldmatrix_x2_trans(r[0], r[1], vc + lm_row_off);
        r[2] = r[3] = 0;
      }
#pragma unroll
      for (int jj = 0; jj < (NBLK >= 2 ? 2 : 1); ++jj) {
        const int blk = bb + jj;
        const uint32_t xl = r[2 * jj], xh = r[2 * jj + 1];
        const uint32_t xl8 = xl >> 8, xh8 = xh >> 8;
#pragma unroll
        for (int pp = 0; pp < P; ++pp) {
          constexpr uint32_t M0 = C::MASK0;
          const uint32_t mask = M0 << (NBITS * pp);
          const int ch = pp * NBLK + blk;
          const int grp = (16 * ch) / GS;
          mma16816(acc[ch], xl & mask, xl8 & mask, xh & mask, xh8 & mask, pb[grp][0],
                   pb[grp][1]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- epilogue: finish the warp's values, merge the warps, store ----
#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    sm_state.l0 += __shfl_xor_sync(kFullMask, sm_state.l0, off);
    sm_state.l1 += __shfl_xor_sync(kFullMask, sm_state.l1, off);
  }
  __syncthreads();  // every warp is done with its ring before it is reused
  float* vals = merge_vals<D>(smem, warp);
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int grp = (16 * ch) / GS;
    const int slice = (16 * ch) / DP;
    const float e = pow2i(24 - NBITS * slice);
    const float z0 = __shfl_sync(kFullMask, zacc[0], grp * 4 + t);
    const float z1 = __shfl_sync(kFullMask, zacc[1], grp * 4 + t);
    // rows g / g+8 of the output tile are dims 16ch+2g / 16ch+2g+1
    float2 h0 = make_float2(fmaf(acc[ch][0], e, z0), fmaf(acc[ch][2], e, z0));
    float2 h1 = make_float2(fmaf(acc[ch][1], e, z1), fmaf(acc[ch][3], e, z1));
    *reinterpret_cast<float2*>(&vals[(2 * t) * D + 16 * ch + 2 * g]) = h0;
    *reinterpret_cast<float2*>(&vals[(2 * t + 1) * D + 16 * ch + 2 * g]) = h1;
  }
  publish_ml<D>(smem, nwarps, warp, lane, sm_state);
  __syncthreads();
  cta_merge_store<D>(p, smem, nwarps, b, hkv, hc, split);
}

// ------------------------------------------------------------------ host side
constexpr int kFusedWarps = 4;
constexpr int kFusedStages = 6;

template <int NBITS, int D, int GS>
struct FusedLaunch {
  static constexpr int STAGES = kFusedStages;
  static int smem_bytes() {
    const int ring = kFusedWarps * STAGES * FusedCfg<NBITS, D, GS>::STAGE_BYTES;
    const int merge = merge_bytes<D>(kFusedWarps);
    return ring > merge ? ring : merge;
  }
  static const void* fn() {
    return reinterpret_cast<const void*>(&fused_split_kernel<NBITS, D, GS, STAGES>);
  }
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
    fused_split_kernel<NBITS, D, GS, STAGES><<<grid, kFusedWarps * 32, smem_bytes(), stream>>>(p);
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
      TKV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn(), kFusedWarps * 32,
                                                             smem_bytes()));
      *ctas = n;
    }
    return TKV_OK;
  }
};

#define TKV_FUSED_DISPATCH(NB, DD, GG, EXPR) \
  if (nbits == NB && D == DD && gs == GG) {  \
    using L = FusedLaunch<NB, DD, GG>;       \
    return EXPR;                             \
  }

#define TKV_FUSED_ALL(EXPR)             \
  TKV_FUSED_DISPATCH(4, 128, 16, EXPR)  \
  TKV_FUSED_DISPATCH(4, 128, 32, EXPR)  \
  TKV_FUSED_DISPATCH(4, 128, 64, EXPR)  \
  TKV_FUSED_DISPATCH(4, 128, 128, EXPR) \
  TKV_FUSED_DISPATCH(2, 128, 16, EXPR)  \
  TKV_FUSED_DISPATCH(2, 128, 32, EXPR)  \
  TKV_FUSED_DISPATCH(2, 128, 64, EXPR)  \
  TKV_FUSED_DISPATCH(2, 128, 128, EXPR) \
  TKV_FUSED_DISPATCH(4, 64, 16, EXPR)   \
  TKV_FUSED_DISPATCH(4, 64, 32, EXPR)   \
  TKV_FUSED_DISPATCH(4, 64, 64, EXPR)   \
  TKV_FUSED_DISPATCH(2, 64, 16, EXPR)   \
  TKV_FUSED_DISPATCH(2, 64, 32, EXPR)   \
  TKV_FUSED_DISPATCH(2, 64, 64, EXPR)

int fused_launch(int nbits, int D, int gs, const DecodeParams& p, cudaStream_t stream) {
  TKV_FUSED_ALL(L::launch(p, stream))
  set_error("fused decode: unsupported (nbits=%d, head_dim=%d, group_size=%d); built: nbits in "
            "{2,4}, head_dim in {64,128}, group_size in {16,32,64,128} with group_size <= head_dim",
            nbits, D, gs);
  return TKV_ERR_UNSUPPORTED;
}

int fused_attrs(int nbits, int D, int gs, int* regs, int* smem, int* local, int* ctas) {
  TKV_FUSED_ALL(L::attrs(regs, smem, local, ctas))
  set_error("fused decode: unsupported (nbits=%d, head_dim=%d, group_size=%d)", nbits, D, gs);
  return TKV_ERR_UNSUPPORTED;
}

}  // namespace tkv

extern "C" int tkv_fused_decode(const void* q, int q_dtype, const uint8_t* k_packed,
                                const void* k_scale, const void* k_zero, const uint8_t* v_packed,
                                const void* v_scale, const void* v_zero, float* acc, float* m,
                                float* l, float* out, int B, int HQ, int HKV, int S, int D,
                                int nbits, int gs, float sm_scale, int num_splits, int split_size,
                                const int32_t* seq_lens, int flags, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(q && k_packed && k_scale && k_zero && v_packed && v_scale && v_zero, TKV_ERR_INVALID,
              "fused decode: null input pointer");
  TKV_REQUIRE(B > 0 && HQ > 0 && HKV > 0 && S > 0, TKV_ERR_INVALID,
              "fused decode: B, HQ, HKV, S must be positive (got %d, %d, %d, %d)", B, HQ, HKV, S);
  TKV_REQUIRE(B <= 65535, TKV_ERR_INVALID, "fused decode: batch %d exceeds 65535", B);
  TKV_REQUIRE(HQ % HKV == 0, TKV_ERR_INVALID, "HQ=%d must be a multiple of HKV=%d", HQ, HKV);
  TKV_REQUIRE(q_dtype >= 0 && q_dtype <= 2, TKV_ERR_INVALID, "fused decode: bad q dtype %d", q_dtype);
  TKV_REQUIRE(num_splits >= 1 && split_size >= 16 && split_size % 16 == 0, TKV_ERR_INVALID,
              "fused decode: split_size=%d must be a positive multiple of 16, num_splits=%d >= 1",
              split_size, num_splits);
  TKV_REQUIRE((int64_t)num_splits * split_size >= S, TKV_ERR_INVALID,
              "fused decode: %d splits of %d tokens do not cover S=%d", num_splits, split_size, S);
  const bool partials = num_splits > 1 || (flags & TKV_FLAG_PARTIALS_ONLY);
  TKV_REQUIRE(!partials || (acc && m && l), TKV_ERR_INVALID,
              "fused decode: partial buffers (acc, m, l) required");
  TKV_REQUIRE(partials || out, TKV_ERR_INVALID, "fused decode: out required");
  TKV_REQUIRE(aligned16(k_packed) && aligned16(v_packed), TKV_ERR_ALIGN,
              "fused decode: packed code pointers must be 16-byte aligned");
  DecodeParams p{};
  p.q = q;
  p.q_dtype = q_dtype;
  p.kp = k_packed;
  p.vp = v_packed;
  p.ks = (const __half*)k_scale;
  p.kz = (const __half*)k_zero;
  p.vs = (const __half*)v_scale;
  p.vz = (const __half*)v_zero;
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
  TKV_REQUIRE((int64_t)HKV * p.hchunks <= 65535, TKV_ERR_INVALID, "fused decode: too many heads");
  const int ng = (gs > 0 && D % gs == 0) ? D / gs : 0;
  p.meta_aligned = (ng > 0 && ((int64_t)S * ng * 2) % 16 == 0 && aligned16(k_scale) &&
                    aligned16(k_zero) && aligned16(v_scale) && aligned16(v_zero))
                       ? 1
                       : 0;
  return fused_launch(nbits, D, gs, p, (cudaStream_t)stream);
}
