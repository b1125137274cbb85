// Fused split-K decode attention on a packed 2/4-bit KV cache (sm_100a).
//
// Replaces _fused_decode_attn_split of the reference (kernels/fused_decode_attn.py:155-353).
//
// Scheduling, the per-warp copy rings and the epilogue live in tkv_splitk_driver.cuh
// (persistent CTAs over balanced tile ranges; one CTA segment serves one (batch, KV
// head, history split) and up to 8 query heads of the GQA group).  This file is the
// tile policy: how a 32-token tile is fetched and what is computed on it.
//
// Data movement.  A stage holds 32 tokens: K codes, V codes, and the four scale/zero
// arrays.  Lane 0 of the warp fetches the codes with two tiled TMA loads; every lane
// fetches a share of the metadata with 16-byte cp.async copies and posts one arrival
// that fires when they land; all of it completes on one mbarrier per stage.  The tensor maps
// view a packed code tensor as rows of 128 bytes (the 32 tokens of a tile are one
// contiguous run) with the hardware 128B swizzle, or -- when sequences do not start on
// 128-byte boundaries -- as [tokens, bytes-per-token] with the 32B/64B swizzle; either
// way the later 8-row x 16-byte ldmatrix reads hit 8 distinct bank groups.  Ragged
// tails and caches whose metadata rows are not 16-byte aligned fetch the metadata with
// plain loads (tokens past the end get scale = zero = 0).  The query rows of a segment
// are staged in shared memory by the driver, one segment ahead.
//
// Arithmetic.  The packed bytes are never expanded to dequantised values.  With
// code c, group scale s and group zero z, a cache value is c*s + z, so
//     q.k = sum_g s_g * (sum_{d in g} q_d c_d)  +  sum_g z_g * (sum_{d in g} q_d)
//     sum_n p_n v_n[d] = sum_n (p_n s_{n,g(d)}) c_n[d]  +  sum_n p_n z_{n,g(d)}
// The inner sums are tensor-core MMAs (m16n8k16, f16 in, f32 accumulate) whose
// A operand is the raw code field, isolated from the packed word by ONE bitwise AND:
// a 2- or 4-bit field inside the mantissa of an f16 is the subnormal (or scaled)
// number c * 2^(pos-24), exact, and the power of two is folded into the f32 scale
// afterwards.  The zero-point terms are one extra MMA each per 16 tokens.
//
// Fragment mapping (g = lane/4, t = lane%4).  Scores use S^T = K Q^T with 16 tokens
// as MMA rows and the 8 heads as columns; the output uses O^T = V^T P^T with 16
// head-dims as rows.  ldmatrix delivers for K the 4 bytes [16b+4t, 16b+4t+4) of
// tokens g / g+8, and with .trans for V the 2 bytes [16b+2g, 16b+2g+2) of token
// pairs (2t, 2t+1) / (2t+8, 2t+9) -- already the layout of an A fragment once masked.
// Chunk ch = slice*NBLK + b covers head dims [16ch, 16ch+16) because of the split-P
// layout (byte j, bit slice p -> dim j + p*DP).
//
// Softmax.  Probabilities are taken relative to a reference exponent m_ref that is
// only raised (to tile max + 4) when a tile exceeds it, so accumulators are rescaled
// a handful of times per split instead of at almost every tile; the true running
// maximum is tracked separately and the partial is converted to it in the epilogue.
#include <cuda.h>

#include "tkv_splitk_driver.cuh"

namespace tkv {

template <int NBITS, int D, int GS, int TOK_ = 32>
struct FusedCfg {
  static constexpr int kTok = TOK_;     // tokens per tile / stage
  static constexpr int MT = kTok / 16;  // 16-token MMA blocks per tile
  static_assert(kTok == 32 || kTok == 64, "a tile is 32 or 64 tokens");
  static constexpr int NBITS_ = NBITS, D_ = D, GS_ = GS;
  static constexpr int P = 8 / NBITS;          // codes per byte = bit slices
  static constexpr int DP = D / P;             // packed bytes per token
  static constexpr int NBLK = DP / 16;         // 16-byte column blocks per token row
  static constexpr int NCH = D / 16;           // 16-dim chunks
  static constexpr int NG = D / GS;            // quantisation groups per token
  static constexpr int ACC_DIMS = GS;  // dims sharing one score accumulator: a quantisation group
  static constexpr int NACC = NG;
  static constexpr int CODE_BYTES = (kTok * DP + 1023) / 1024 * 1024;  // keeps V's swizzle phase
  static constexpr int NPAIR = (NBLK + 1) / 2;  // ldmatrix issues per 16-token half
  static constexpr int META_BYTES = kTok * NG * 2;
  // Distance between the four metadata arrays of a stage.  With one group per token a row
  // is 2 bytes and a tile may start 2 bytes off a 4-byte boundary: such tiles are copied
  // from the boundary below (one 4-byte copy more) and read back at a 2-byte shift, which
  // is kept in the word after the arrays.
  static constexpr int META_STRIDE = (NG == 1) ? META_BYTES + 16 : META_BYTES;
  static constexpr int SHIFT_WORD = 4 * META_STRIDE;  // byte offset inside the metadata area
  static constexpr int PAYLOAD = 2 * CODE_BYTES + 4 * META_STRIDE + (NG == 1 ? 16 : 0);
  static constexpr int MERGE_BYTES = kHeadsPerCta * D * 4;  // one warp's partial in the epilogue
  static constexpr int STAGE_BYTES =
      ((PAYLOAD > MERGE_BYTES ? PAYLOAD : MERGE_BYTES) + 1023) / 1024 * 1024;  // keeps swizzle atoms aligned
  static constexpr uint32_t MASK0 = ((1u << NBITS) - 1u) * 0x00010001u;
  static constexpr int SWZ_SHIFT = (NBLK == 4) ? 1 : 2;
  static_assert(NBLK == 1 || NBLK == 2 || NBLK == 4, "packed row must be 16, 32 or 64 bytes");
  static_assert(GS >= 16 && NG >= 1 && NG <= 8, "group size must be 16..D with at most 8 groups");
};

// Device-side status word: 0 = ok, 1 = a bounded mbarrier wait gave up.
__device__ int g_fused_status;

template <int NG>
struct MetaRow {
  uint32_t w[(NG + 1) / 2];  // NG halves
};
template <int NG>
__device__ __forceinline__ MetaRow<NG> lds_meta_row(uint32_t addr) {
  MetaRow<NG> r;
  if constexpr (NG == 8) {
    const uint4 v = lds_v4(addr);
    r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
  } else if constexpr (NG == 4) {
    const uint2 v = lds_v2(addr);
    r.w[0] = v.x; r.w[1] = v.y;
  } else if constexpr (NG == 2) {
    r.w[0] = lds_u32(addr);
  } else {
    r.w[0] = lds_u16(addr);
  }
  return r;
}
template <int NG>
__device__ __forceinline__ float meta_f32(const MetaRow<NG>& r, int i) {
  const __half2 h = *reinterpret_cast<const __half2*>(&r.w[i >> 1]);
  return (i & 1) ? __high2float(h) : __low2float(h);
}
// {x_i, x_i} as a half2 register operand (folds into the multiply's operand selector)
template <int NG>
__device__ __forceinline__ __half2 meta_bcast(const MetaRow<NG>& r, int i) {
  const __half2 h = *reinterpret_cast<const __half2*>(&r.w[i >> 1]);
  return (i & 1) ? __high2half2(h) : __low2half2(h);
}


// A16: every scale/zero tile starts on a 16-byte boundary (the common case).  The other
// instantiation serves caches whose rows start on smaller boundaries; keeping the two apart
// keeps each kernel's instruction footprint small (a decode kernel usually starts with a
// cold instruction cache, and the copy code is inlined at three places).
// KCHAN: the K scale/zero arrays hold one row of D values per block of kTok tokens (keys
// quantised per channel over groups of kTok tokens) instead of D/GS values per token.  With
// GS == kTok both forms fill the same bytes of a stage, so only the source address of the two
// K metadata copies and the score arithmetic differ.
template <int NBITS, int D_, int GS, bool A16 = true, int TOK_ = 32, int WARPS_ = 4, int STAGES_ = 3,
          int MIN_CTAS_ = 3, bool PIPELINED_ = true, bool KCHAN_ = false>
struct FusedPolicy {
  using C = FusedCfg<NBITS, D_, GS, TOK_>;
  static constexpr bool KCHAN = KCHAN_;
  static_assert(!KCHAN || (GS == TOK_ && A16 && D_ / GS > 1),
                "per-channel keys: value groups of one tile's tokens, 16-byte aligned rows");
  static constexpr int D = D_;
  static constexpr int kTok = C::kTok, MT = C::MT;
  static constexpr int TOK = kTok;
  static constexpr bool PIPELINED = PIPELINED_;
  static constexpr int WARPS = WARPS_;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int STAGE_BYTES = C::STAGE_BYTES;
  // arrivals per stage: lane 0's expect_tx for the code tiles + one per lane for the metadata
  static constexpr int BAR_COUNT = 33;
  static constexpr int P = C::P, DP = C::DP, NBLK = C::NBLK, NCH = C::NCH, NG = C::NG;
  static constexpr int NACC = C::NACC, ACC_DIMS = C::ACC_DIMS;

  struct Maps {
    CUtensorMap k, v;  // with kv_one: `k` spans both tensors and `v` is unused
  };
  struct Query {
    uint32_t qf[NCH][2];  // B operand of the score MMA; bit slice p is pre-scaled by 2^(-NBITS p)
    uint32_t qz0, qz1;    // B operand of the K zero-point MMA: f16 hi / lo parts of
                          // qk_scale * (sum of q over a group), groups 2t and 2t+1
    uint32_t off[MT][C::NPAIR];  // this lane's ldmatrix byte offsets inside a code tile
    uint32_t o_row;   // byte offset of token g's row inside a scale array
    uint32_t o_kz;    // byte offset of this lane's K zero-point word (token g)
    uint32_t o_vz;    // byte offset of this lane's first V zero-point (token 2t, group g mod NG)
    uint32_t ones;    // (1, 1) in f16 on lanes 0-3: row 8 of the zero-point MMA sums the p's
    uint32_t kofs, vofs;  // where the K and the V tile sit inside a stage
  };
  struct Accum {
    float m_ref0, m_ref1;    // exponent the probabilities refer to (same on the 8 lanes of a head)
    float m_true0, m_true1;  // this lane's running maxima (reduced over lanes in finalize)
    float acc[NCH][4];
    float zacc[4];  // rows 0..NG-1: sum_n p_n z_n[group]; row 8: sum_n p_n
  };

  __device__ static void report_timeout() { atomicExch(&g_fused_status, 1); }
  __device__ static __forceinline__ void prefetch_maps(const Maps& maps) {
    prefetch_tensormap(&maps.k);
    prefetch_tensormap(&maps.v);
  }

  // Per-lane constants of the copy path, set once per warp.
  static constexpr int CPA = C::META_BYTES / 16;                   // 16-byte chunks per metadata array
  static constexpr int ROUNDS = (4 * CPA + 31) / 32;               // cp.async rounds per tile
  struct IssueState {
    const uint8_t* src[ROUNDS];  // this lane's source of round r at global row 0
    bool is_k[ROUNDS];           // the chunk belongs to the K scale or zero array
  };
  __device__ static __forceinline__ void issue_init(IssueState& is, const DecodeParams& p, int lane) {
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
      const int i = r * 32 + lane;              // chunk index over (ks | kz | vs | vz)
      const int arr = (i / CPA) & 3, c = i % CPA;
      const __half* base = arr == 0 ? p.ks : arr == 1 ? p.kz : arr == 2 ? p.vs : p.vz;
      is.src[r] = reinterpret_cast<const uint8_t*>(base) + c * 16;
      is.is_k[r] = arr < 2;
    }
  }

  // Fill one stage with the 32 tokens starting at global row `row`; `nvalid` of them
  // belong to the unit.
  __device__ static __forceinline__ void issue(const IssueState& is, const DecodeParams& p,
                                               const Maps& maps, int row, int nvalid, uint32_t st,
                                               uint8_t* st_ptr, uint32_t bar, int lane) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, 2 * kTok * DP);
      // wide view: the tensor is [bytes/128, 128]; narrow view: [tokens, DP]
      constexpr int SH = (DP == 64) ? 1 : (DP == 32) ? 2 : 3;  // row*DP/128 = row >> SH
      const int c1 = p.wide ? (row >> SH) : row;
      if (p.kv_one) {
        tma_load_3d(st, &maps.k, 0, c1, 0, bar);
      } else {
        tma_load_2d(st, &maps.k, 0, c1, bar);
        tma_load_2d(st + C::CODE_BYTES, &maps.v, 0, c1, bar);
      }
    }
    // Scale/zero: 16-byte cp.async per lane (a bulk-copy instruction costs the issuing warp
    // ~100+ cycles each, four of them per tile were a third of the loop time); every lane
    // then posts one arrival on the stage barrier that fires when its copies have landed.
    const uint32_t mst = st + 2 * C::CODE_BYTES;
    if constexpr (A16) {
      if (NG == 1 && lane == 0)  // no read-back shift (see FusedCfg::META_STRIDE)
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(mst + C::SHIFT_WORD), "r"(0u) : "memory");
      if (KCHAN || (NG > 1 && nvalid == kTok)) {
        const int64_t off = (int64_t)row * (NG * 2);  // bytes
        // per-channel keys: one (D,) row per tile; tiles start on multiples of kTok tokens
        const int64_t off_k = KCHAN ? (int64_t)(row / kTok) * (D * 2) : off;
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
          if (4 * CPA >= 32 || lane < 4 * CPA)
            cp_async16(mst + (r * 32 + lane) * 16, is.src[r] + ((KCHAN && is.is_k[r]) ? off_k : off), 16);
        }
        cp_async_mbar_arrive_noinc(bar);
      } else {
        issue_meta<16>(p, row, nvalid, mst, bar, lane);
      }
    } else if constexpr (NG >= 4) {
      issue_meta<8>(p, row, nvalid, mst, bar, lane);   // rows of 8 or 16 bytes
    } else if constexpr (NG == 2) {
      issue_meta<4>(p, row, nvalid, mst, bar, lane);   // rows of 4 bytes
    } else {
      // one group per row: rows are aligned to 2 bytes only.  Copy from the 4-byte boundary
      // below and let the reader skip the first `shift` bytes (0 when the tile is aligned).
      const int shift = (p.meta_phase + row * 2) & 3;  // 0 or 2
      if (lane == 0)
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(mst + C::SHIFT_WORD), "r"((uint32_t)shift)
                     : "memory");
      constexpr int N = C::META_BYTES / 4 + 1;  // 4-byte copies per array
      const int vbytes = nvalid * NG * 2 + shift;
      const int64_t off = (int64_t)row * (NG * 2) - shift;
      for (int i = lane; i < 4 * N; i += 32) {
        const int arr = i / N, c = i - arr * N;
        const uint8_t* base = reinterpret_cast<const uint8_t*>(
            arr == 0 ? p.ks : arr == 1 ? p.kz : arr == 2 ? p.vs : p.vz);
        const int nb = min(max(vbytes - c * 4, 0), 4);
        cp_async_n<4>(mst + arr * C::META_STRIDE + c * 4, nb > 0 ? base + off + c * 4 : base - p.meta_phase,
                      nb);
      }
      cp_async_mbar_arrive_noinc(bar);
    }
    (void)st_ptr;
  }

  // Scale/zero of a tile in CS-byte copies: rows that only start on 8- or 4-byte boundaries
  // (odd history lengths), and the last tile of a unit, whose tokens past the end are
  // zero-filled by the copy itself (scale = zero = 0 makes them contribute exact zeros).
  template <int CS>
  __device__ static __forceinline__ void issue_meta(const DecodeParams& p, int row, int nvalid,
                                                    uint32_t mst, uint32_t bar, int lane) {
    constexpr int N = C::META_BYTES / CS;  // copies per array
    const int vbytes = nvalid * NG * 2;    // valid bytes of each array in this tile
    const int64_t off = (int64_t)row * (NG * 2);
#pragma unroll
    for (int i0 = 0; i0 < 4 * N; i0 += 32) {
      const int i = i0 + lane;
      if (4 * N >= 32 || i < 4 * N) {
        const int arr = (i / N) & 3, c = i % N;
        const uint8_t* base = reinterpret_cast<const uint8_t*>(
            arr == 0 ? p.ks : arr == 1 ? p.kz : arr == 2 ? p.vs : p.vz);
        const int nb = min(max(vbytes - c * CS, 0), CS);
        cp_async_n<CS>(mst + arr * C::META_STRIDE + c * CS, nb > 0 ? base + off + c * CS : base, nb);
      }
    }
    cp_async_mbar_arrive_noinc(bar);
  }

  // Lane constants of the tile loop: set once per warp.
  __device__ static __forceinline__ void lane_init(Query& qq, const DecodeParams& p, int lane) {
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix addressing: lane l supplies the row address of matrix l/8, row l%8;
    // matrices are (tokens 0-7, blk), (tokens 8-15, blk), (tokens 0-7, blk+1), (tokens 8-15, blk+1).
    const int lm_r = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int lm_b = (NBLK >= 2) ? (lane >> 4) : 0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int pr = 0; pr < C::NPAIR; ++pr) {
        const int n = 16 * mt + lm_r, blk = 2 * pr + lm_b;
        const int L = n * NBLK + blk;  // linear 16-byte chunk index inside the tile
        int Ls;
        if (p.wide) {
          Ls = (L & ~7) | ((L ^ (L >> 3)) & 7);                       // 128B swizzle
        } else {
          const int swz = (NBLK > 1) ? ((n >> C::SWZ_SHIFT) & (NBLK - 1)) : 0;
          Ls = n * NBLK + (blk ^ swz);                                // 32B / 64B swizzle
        }
        qq.off[mt][pr] = Ls << 4;
      }
    qq.o_row = g * NG * 2;
    qq.o_kz = (NG >= 2) ? (g * NG + ((2 * t) % NG)) * 2 : g * 2;
    qq.o_vz = ((2 * t) * NG + (g % NG)) * 2;
    qq.ones = (lane < 4) ? 0x3C003C00u : 0u;
    qq.kofs = (p.kv_one && p.k_second) ? C::CODE_BYTES : 0;
    qq.vofs = C::CODE_BYTES - qq.kofs;
  }

  // Query fragments of a segment are the same for the four warps: each warp builds the
  // chunks w, w+WARPS, ... and the per-chunk sums of q, the CTA synchronises, and every
  // warp reads the finished fragments (layout [word quad][lane], conflict free).
  static constexpr int QFRAG_WORDS = NCH * 2;                        // per lane
  static constexpr int QFRAG_BYTES = 32 * QFRAG_WORDS * 4 + NCH * 8 * 4;  // fragments + chunk sums
  static_assert(QFRAG_WORDS % 4 == 0, "fragments are read as 128-bit words");

  // `qsm`: the segment's 8 query rows (raw dtype, zero rows for heads past the group)
  __device__ static __forceinline__ void build_query(const DecodeParams& p, const uint8_t* qsm,
                                                     uint32_t qfrag, int warp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* qrow = qsm + g * D * (p.q_dtype == TKV_DTYPE_F32 ? 4 : 2);
    const uint32_t qrow_s = smem_u32(qrow);
#pragma unroll
    for (int c0 = 0; c0 < NCH; c0 += WARPS) {
      const int ch = c0 + warp;
      if (NCH % WARPS != 0 && ch >= NCH) break;
      __half x[4];
      if (p.q_dtype == TKV_DTYPE_F16) {
        const uint2 v = lds_v2(qrow_s + (16 * ch + 4 * t) * 2);
        *reinterpret_cast<uint2*>(x) = v;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = load_q_half(qrow, p.q_dtype, 16 * ch + 4 * t + i);
      }
      // The code field of bit slice p is the f16 number c * 2^(NBITS p - 24); scaling the
      // query down by the same power of two (exact unless |q| < 2^-14 2^(NBITS p), where the
      // absolute error stays below 2^-25) lets every slice share one accumulator and scale.
      const int slice = ch / NBLK;
      const __half2 down = __float2half2_rn(ex2((float)(-NBITS * slice)));
      const uint32_t u0 = pack_half2(x[0], x[2]);  // k-slots 2t, 2t+1   <-> dims 16ch+4t, 16ch+4t+2
      const uint32_t u1 = pack_half2(x[1], x[3]);  // k-slots 2t+8, 2t+9 <-> dims 16ch+4t+1, 16ch+4t+3
      const __half2 v0 = __hmul2(*reinterpret_cast<const __half2*>(&u0), down);
      const __half2 v1 = __hmul2(*reinterpret_cast<const __half2*>(&u1), down);
      float sum = (__half2float(x[0]) + __half2float(x[1])) + (__half2float(x[2]) + __half2float(x[3]));
      sum += __shfl_xor_sync(kFullMask, sum, 1);
      sum += __shfl_xor_sync(kFullMask, sum, 2);
      // words (2ch, 2ch+1) of this lane: quad ch/2, position 2(ch%2)
      const uint32_t dst = qfrag + (ch >> 1) * 512 + lane * 16 + (ch & 1) * 8;
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(dst),
                   "r"(*reinterpret_cast<const uint32_t*>(&v0)),
                   "r"(*reinterpret_cast<const uint32_t*>(&v1))
                   : "memory");
      if (t == 0)
        asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(qfrag + 32 * QFRAG_WORDS * 4 + (ch * 8 + g) * 4),
                     "f"(sum)
                     : "memory");
    }
  }

  // After the CTA barrier that follows build_query.
  __device__ static __forceinline__ void load_query(Query& qq, const DecodeParams& p,
                                                    const uint8_t*, uint32_t qfrag, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int q4 = 0; q4 < QFRAG_WORDS / 4; ++q4) {
      const uint4 v = lds_v4(qfrag + q4 * 512 + lane * 16);
      qq.qf[2 * q4][0] = v.x;
      qq.qf[2 * q4][1] = v.y;
      qq.qf[2 * q4 + 1][0] = v.z;
      qq.qf[2 * q4 + 1][1] = v.w;
    }
    // k-slots 2t, 2t+1 carry the f16 high parts of qk_scale * (sum of q over groups 2t, 2t+1)
    // for head g, k-slots 2t+8, 2t+9 the low parts (the zero-point words feed both halves).
    constexpr int CPG = GS / 16;  // chunks per group
    const uint32_t sums = qfrag + 32 * QFRAG_WORDS * 4 + g * 4;
    __half hi[2], lo[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int grp = 2 * t + k;
      float v = 0.f;
      if (grp < NG) {
#pragma unroll
        for (int c = 0; c < CPG; ++c) {
          float x;
          asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(x) : "r"(sums + ((grp * CPG + c) * 8) * 4));
          v += x;
        }
      }
      v *= p.qk_scale;
      hi[k] = __float2half_rn(v);
      lo[k] = __float2half_rn(v - __half2float(hi[k]));
    }
    qq.qz0 = pack_half2(hi[0], hi[1]);
    qq.qz1 = pack_half2(lo[0], lo[1]);
  }

  __device__ static __forceinline__ void reset(Accum& ac) {
    ac.m_ref0 = ac.m_ref1 = ac.m_true0 = ac.m_true1 = -INFINITY;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
      for (int i = 0; i < 4; ++i) ac.acc[ch][i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) ac.zacc[i] = 0.f;
  }

  struct Scores {
    float s[MT][4];  // [16-token block][(token g, head 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)]
  };

  // Scores of one tile in stage `st` (scaled by qk_scale, tokens past the unit
  // end set to -inf); `left` = tokens from the tile start to the unit end.
  // Per-channel keys: K = code * s[d] + z[d] with one (s, z) row for the whole tile, so
  //     q.k_n = sum_d (q_d s_d) c_{n,d} + sum_d q_d z_d.
  // The scale goes into the B operand, formed per chunk as an f16 pair hi + lo with
  // hi = rn(q s) and lo = fma(q, s, -hi), the exact rounding error of hi -- an outlier channel
  // has a large s, and q s rounded to f16 once would put 2^-11 of the largest terms into
  // every score.  All chunks share ONE accumulator per 16 tokens, and the zero-point term --
  // the same for every token of the tile -- is one MMA per chunk whose A operand is the z
  // row repeated down the token rows.
  __device__ static __forceinline__ void scores_kchan(Scores& out, const Query& qq, uint32_t st,
                                                      int left, float qk_scale, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kc = st + qq.kofs;
    const uint32_t ms = st + 2 * C::CODE_BYTES;
    const uint32_t ks_r = ms + t * 8;                     // dims 16ch + 4t .. 16ch + 4t + 3 of a chunk
    const uint32_t kz_r = ms + C::META_STRIDE + t * 8;
    const float qk24 = qk_scale * 16777216.f;  // the code fields carry 2^-24
    float cz[4];
    float c[MT][4];
    bool started = false;  // resolved at compile time: the loops below are fully unrolled
#pragma unroll
    for (int bb = 0; bb < NBLK; bb += 2) {
      uint32_t r[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if constexpr (NBLK >= 2) {
          ldmatrix_x4(r[mt], kc + qq.off[mt][bb >> 1]);
        } else {
          ldmatrix_x2(r[mt][0], r[mt][1], kc + qq.off[mt][0]);
          r[mt][2] = r[mt][3] = 0;
        }
      }
#pragma unroll
      for (int jj = 0; jj < (NBLK >= 2 ? 2 : 1); ++jj) {
        const int blk = bb + jj;
#pragma unroll
        for (int pp = 0; pp < P; ++pp) {
          constexpr uint32_t M0 = C::MASK0;
          const uint32_t mask = M0 << (NBITS * pp);
          const int ch = pp * NBLK + blk;
          // ---- this chunk's B operands: q s as hi + lo, and the z row against q ----
          const uint2 sv = lds_v2(ks_r + ch * 32);
          const uint2 zv = lds_v2(kz_r + ch * 32);
          // k-slots 2t, 2t+1 <-> dims 16ch+4t, 16ch+4t+2; k-slots 2t+8, 2t+9 <-> dims +1, +3
          const uint32_t s02 = __byte_perm(sv.x, sv.y, 0x5410), s13 = __byte_perm(sv.x, sv.y, 0x7632);
          uint32_t z02 = __byte_perm(zv.x, zv.y, 0x5410), z13 = __byte_perm(zv.x, zv.y, 0x7632);
          const uint32_t hi0 = hmul2_u32(qq.qf[ch][0], s02), hi1 = hmul2_u32(qq.qf[ch][1], s13);
          const uint32_t lo0 = hfma2_u32(qq.qf[ch][0], s02, hi0 ^ 0x80008000u);
          const uint32_t lo1 = hfma2_u32(qq.qf[ch][1], s13, hi1 ^ 0x80008000u);
          if (pp > 0) {  // the query of bit slice p carries 2^(-NBITS p): the zero row takes it back
            const __half2 up2 = __float2half2_rn(pow2i(NBITS * pp));
            const uint32_t up = *reinterpret_cast<const uint32_t*>(&up2);
            z02 = hmul2_u32(z02, up);
            z13 = hmul2_u32(z13, up);
          }
          if (!started) {
            mma16816_zero(cz, z02, z02, z13, z13, qq.qf[ch][0], qq.qf[ch][1]);
          } else {
            mma16816(cz, z02, z02, z13, z13, qq.qf[ch][0], qq.qf[ch][1]);
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t xl = r[mt][2 * jj], xh = r[mt][2 * jj + 1];
            const uint32_t a0 = xl & mask, a1 = xh & mask, a2 = (xl >> 8) & mask, a3 = (xh >> 8) & mask;
            if (!started) {
              mma16816_zero(c[mt], a0, a1, a2, a3, hi0, hi1);
            } else {
              mma16816(c[mt], a0, a1, a2, a3, hi0, hi1);
            }
            mma16816(c[mt], a0, a1, a2, a3, lo0, lo1);
          }
          started = true;
        }
      }
    }
    float (&sc)[MT][4] = out.s;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[mt][i] = fmaf(c[mt][i], qk24, cz[i] * qk_scale);
    if (left < kTok) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (mt * 16 + g >= left) sc[mt][0] = sc[mt][1] = -INFINITY;
        if (mt * 16 + g + 8 >= left) sc[mt][2] = sc[mt][3] = -INFINITY;
      }
    }
  }

  __device__ static __forceinline__ void scores(Scores& out, const Query& qq, uint32_t st,
                                                const uint8_t*, int left, float qk_scale,
                                                int lane) {
    if constexpr (KCHAN) {
      scores_kchan(out, qq, st, left, qk_scale, lane);
      return;
    }
    const int g = lane >> 2;
    const uint32_t kc = st + qq.kofs;
    uint32_t ms = st + 2 * C::CODE_BYTES;
    if constexpr (NG == 1) ms += lds_u32(ms + C::SHIFT_WORD);  // 0 or 2, see FusedCfg::META_STRIDE
    const uint32_t ks_a = ms + qq.o_row;
    const uint32_t kz_a = ms + C::META_STRIDE + qq.o_kz;
    const float qk24 = qk_scale * 16777216.f;  // the code fields carry 2^-24
    constexpr int HALF = 16 * NG * 2;           // bytes of 16 token rows in a metadata array

    float (&sc)[MT][4] = out.s;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float c[NACC][4];
      bool started[NACC];  // resolved at compile time: the loops below are fully unrolled
#pragma unroll
      for (int a = 0; a < NACC; ++a) started[a] = false;
#pragma unroll
      for (int bb = 0; bb < NBLK; bb += 2) {
        uint32_t r[4];
        if constexpr (NBLK >= 2) {
          ldmatrix_x4(r, kc + qq.off[mt][bb >> 1]);
        } else {
          ldmatrix_x2(r[0], r[1], kc + qq.off[mt][0]);
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
            const int a = (16 * ch) / ACC_DIMS;
            if (!started[a]) {
              mma16816_zero(c[a], xl & mask, xh & mask, xl8 & mask, xh8 & mask, qq.qf[ch][0],
                            qq.qf[ch][1]);
              started[a] = true;
            } else {
              mma16816(c[a], xl & mask, xh & mask, xl8 & mask, xh8 & mask, qq.qf[ch][0],
                       qq.qf[ch][1]);
            }
          }
        }
      }
      // zero-point term (already times qk_scale): sum_g z[token][g] * qsum[g][head].  The
      // word holding (z[2t], z[2t+1]) feeds k-slots 2t, 2t+1 (against the high parts) and
      // 2t+8, 2t+9 (against the low parts); lanes past the last group re-read a valid word
      // against a zero B operand.
      float s4[4];
      {
        uint32_t zl, zh;
        if constexpr (NG >= 2) {
          zl = lds_u32(kz_a + mt * HALF);
          zh = lds_u32(kz_a + mt * HALF + HALF / 2);
        } else {
          zl = lds_u16(kz_a + mt * HALF);
          zh = lds_u16(kz_a + mt * HALF + HALF / 2);
        }
        mma16816_zero(s4, zl, zh, zl, zh, qq.qz0, qq.qz1);
      }
      // scale term
      {
        const MetaRow<NG> s_lo = lds_meta_row<NG>(ks_a + mt * HALF);
        const MetaRow<NG> s_hi = lds_meta_row<NG>(ks_a + mt * HALF + HALF / 2);
        float t4[4];
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          const float f_lo = meta_f32<NG>(s_lo, a);
          const float f_hi = meta_f32<NG>(s_hi, a);
          if (a == 0) {
            t4[0] = c[a][0] * f_lo;
            t4[1] = c[a][1] * f_lo;
            t4[2] = c[a][2] * f_hi;
            t4[3] = c[a][3] * f_hi;
          } else {
            t4[0] = fmaf(c[a][0], f_lo, t4[0]);
            t4[1] = fmaf(c[a][1], f_lo, t4[1]);
            t4[2] = fmaf(c[a][2], f_hi, t4[2]);
            t4[3] = fmaf(c[a][3], f_hi, t4[3]);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[mt][i] = fmaf(t4[i], qk24, s4[i]);
      }
    }
    if (left < kTok) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (mt * 16 + g >= left) sc[mt][0] = sc[mt][1] = -INFINITY;
        if (mt * 16 + g + 8 >= left) sc[mt][2] = sc[mt][3] = -INFINITY;
      }
    }
  }

  // Online softmax update and O^T += V^T P^T for the tile whose scores are `in`.
  __device__ static __forceinline__ void update(Accum& ac, const Query& qq, Scores& in,
                                                uint32_t st, uint8_t*, int left, int lane) {
    const uint32_t vc = st + qq.vofs;
    uint32_t ms = st + 2 * C::CODE_BYTES;
    if constexpr (NG == 1) ms += lds_u32(ms + C::SHIFT_WORD);
    const uint32_t vs_a = ms + 2 * C::META_STRIDE + qq.o_row;
    const uint32_t vz_a = ms + 3 * C::META_STRIDE + qq.o_vz;
    constexpr int HALF = 16 * NG * 2;
    float (&sc)[MT][4] = in.s;
    // ---- online softmax with a lazily raised reference exponent ----
    {
      // this lane's maxima for heads 2t / 2t+1; the cross-lane maximum is only needed
      // when some lane exceeds the reference (rare) and in finalize
      float mx0 = fmaxf(sc[0][0], sc[0][2]);
      float mx1 = fmaxf(sc[0][1], sc[0][3]);
#pragma unroll
      for (int mt = 1; mt < MT; ++mt) {
        mx0 = fmaxf(mx0, fmaxf(sc[mt][0], sc[mt][2]));
        mx1 = fmaxf(mx1, fmaxf(sc[mt][1], sc[mt][3]));
      }
      ac.m_true0 = fmaxf(ac.m_true0, mx0);
      ac.m_true1 = fmaxf(ac.m_true1, mx1);
      if (__any_sync(kFullMask, (mx0 > ac.m_ref0) || (mx1 > ac.m_ref1))) {
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, off));
          mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, off));
        }
        const float n0 = (mx0 > ac.m_ref0) ? mx0 + kLazyTau : ac.m_ref0;
        const float n1 = (mx1 > ac.m_ref1) ? mx1 + kLazyTau : ac.m_ref1;
        const float alpha0 = ex2(ac.m_ref0 - n0);  // first tile: 2^(-inf) = 0; unchanged: 1
        const float alpha1 = ex2(ac.m_ref1 - n1);
        ac.m_ref0 = n0;
        ac.m_ref1 = n1;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          ac.acc[ch][0] *= alpha0;
          ac.acc[ch][1] *= alpha1;
          ac.acc[ch][2] *= alpha0;
          ac.acc[ch][3] *= alpha1;
        }
        ac.zacc[0] *= alpha0;
        ac.zacc[1] *= alpha1;
        ac.zacc[2] *= alpha0;
        ac.zacc[3] *= alpha1;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        sc[mt][0] = ex2(sc[mt][0] - ac.m_ref0);
        sc[mt][1] = ex2(sc[mt][1] - ac.m_ref1);
        sc[mt][2] = ex2(sc[mt][2] - ac.m_ref0);
        sc[mt][3] = ex2(sc[mt][3] - ac.m_ref1);
      }
    }

    // ---- output: O^T += V^T P^T ----
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const uint32_t ph_lo = pack_half2(sc[mt][0], sc[mt][1]);  // token g,   heads 2t, 2t+1
      const uint32_t ph_hi = pack_half2(sc[mt][2], sc[mt][3]);  // token g+8
      {
        // zero-point term: rows = groups, k = tokens, B = unscaled P^T.  Lanes whose g is
        // not a group re-read group g mod NG (those output rows are never used); row 8 is
        // all ones on its k-slots and so accumulates sum_n p_n.
        const uint32_t pz0 = movmatrix_trans(ph_lo);
        const uint32_t pz1 = movmatrix_trans(ph_hi);
        const uint32_t b = vz_a + mt * HALF;
        const uint32_t a0 = lds_u16(b) | (lds_u16(b + NG * 2) << 16);
        const uint32_t a2 = lds_u16(b + HALF / 2) | (lds_u16(b + HALF / 2 + NG * 2) << 16);
        mma16816(ac.zacc, a0, qq.ones, a2, qq.ones, pz0, pz1);
      }
      uint32_t pb[NG][2];
      {
        const MetaRow<NG> s_lo = lds_meta_row<NG>(vs_a + mt * HALF);
        const MetaRow<NG> s_hi = lds_meta_row<NG>(vs_a + mt * HALF + HALF / 2);
        const __half2 p_lo = *reinterpret_cast<const __half2*>(&ph_lo);
        const __half2 p_hi = *reinterpret_cast<const __half2*>(&ph_hi);
#pragma unroll
        for (int grp = 0; grp < NG; ++grp) {
          const __half2 a = __hmul2(p_lo, meta_bcast<NG>(s_lo, grp));
          const __half2 bq = __hmul2(p_hi, meta_bcast<NG>(s_hi, grp));
          pb[grp][0] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&a));
          pb[grp][1] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&bq));
        }
      }
#pragma unroll
      for (int bb = 0; bb < NBLK; bb += 2) {
        uint32_t r[4];
        if constexpr (NBLK >= 2) {
          ldmatrix_x4_trans(r, vc + qq.off[mt][bb >> 1]);
        } else {
          ldmatrix_x2_trans(r[0], r[1], vc + qq.off[mt][0]);
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
            mma16816(ac.acc[ch], xl & mask, xl8 & mask, xh & mask, xh8 & mask, pb[grp][0],
                     pb[grp][1]);
          }
        }
      }
    }
    (void)left;
    (void)lane;
  }

  // Reduce the warp's state, convert it from the reference exponent to the true
  // maximum (the partial format has m = max) and write vals[head][dim] (8 x D floats).
  __device__ static __forceinline__ void finalize(Accum& ac, float* vals, SoftmaxState& st,
                                                  int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
      ac.m_true0 = fmaxf(ac.m_true0, __shfl_xor_sync(kFullMask, ac.m_true0, off));
      ac.m_true1 = fmaxf(ac.m_true1, __shfl_xor_sync(kFullMask, ac.m_true1, off));
    }
    // row 8 of the zero-point accumulator (lanes 0-3, registers 2 and 3) holds sum_n p_n
    const float l0 = __shfl_sync(kFullMask, ac.zacc[2], t);
    const float l1 = __shfl_sync(kFullMask, ac.zacc[3], t);
    const float f0 = (ac.m_true0 == -INFINITY) ? 0.f : ex2(ac.m_ref0 - ac.m_true0);
    const float f1 = (ac.m_true1 == -INFINITY) ? 0.f : ex2(ac.m_ref1 - ac.m_true1);
    st = SoftmaxState{ac.m_true0, ac.m_true1, l0 * f0, l1 * f1};
    const uint32_t vals_s = smem_u32(vals);
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int grp = (16 * ch) / GS;
      const int slice = (16 * ch) / DP;
      const float e = pow2i(24 - NBITS * slice);
      const float z0 = __shfl_sync(kFullMask, ac.zacc[0], grp * 4 + t);
      const float z1 = __shfl_sync(kFullMask, ac.zacc[1], grp * 4 + t);
      // rows g / g+8 of the output tile are dims 16ch+2g / 16ch+2g+1
      sts_v2f(vals_s + ((2 * t) * D + 16 * ch + 2 * g) * 4, fmaf(ac.acc[ch][0], e, z0) * f0,
              fmaf(ac.acc[ch][2], e, z0) * f0);
      sts_v2f(vals_s + ((2 * t + 1) * D + 16 * ch + 2 * g) * 4, fmaf(ac.acc[ch][1], e, z1) * f1,
              fmaf(ac.acc[ch][3], e, z1) * f1);
    }
  }
};

// ------------------------------------------------------------------ host side
// Two kernel families per (nbits, head_dim, group_size, row alignment):
//  * batched -- 4 warps, ring of 3 stages, software-pipelined tile loop, 3 CTAs per SM: the
//    balanced schedules (modes 1 and 3), where a CTA streams tens of tiles per warp;
//  * long -- 8 warps, ring of 2 stages, one tile at a time, 2 CTAs per SM: few long units
//    (mode 2: small batches, and the static one-CTA-per-unit plan).  The same 16 warps per SM
//    in two thirds of the CTAs: a third fewer partial slots for the merge that follows and a
//    third fewer query loads and epilogues, which is what a step of 2-3 tiles per warp is
//    made of (measured: batch 1, ctx 65536, 4-bit step 12.4 -> 10.8 us).
constexpr int kVariantBatched = 0, kVariantLong = 1;
template <int NB, int DD, int GG, bool A16, bool KCHAN = false>
using BatchedPolicy = FusedPolicy<NB, DD, GG, A16, 32, 4, 3, 3, true, KCHAN>;
template <int NB, int DD, int GG, bool A16, bool KCHAN = false>
using LongPolicy = FusedPolicy<NB, DD, GG, A16, 32, 8, 2, 2, false, KCHAN>;

// Keys quantised per channel (value groups of 32): dense batches only, so mode 1 and mode 2.
#define TKV_KCHAN_DISPATCH(NB, DD, EXPR)                            \
  if (nbits == NB && D == DD && gs == 32) {                         \
    using PB = BatchedPolicy<NB, DD, 32, true, true>;               \
    using PL = LongPolicy<NB, DD, 32, true, true>;                  \
    using LB = SplitLaunch<PB, 0x2>;                                \
    using LL = SplitLaunch<PL, 0x4>;                                \
    return EXPR;                                                    \
  }
#define TKV_KCHAN_ALL(EXPR)        \
  TKV_KCHAN_DISPATCH(4, 128, EXPR) \
  TKV_KCHAN_DISPATCH(2, 128, EXPR) \
  TKV_KCHAN_DISPATCH(4, 64, EXPR)  \
  TKV_KCHAN_DISPATCH(2, 64, EXPR)

#define TKV_FUSED_DISPATCH(NB, DD, GG, EXPR)                        \
  if (nbits == NB && D == DD && gs == GG) {                         \
    if (aligned16_rows) {                                           \
      using PB = BatchedPolicy<NB, DD, GG, true>;                   \
      using PL = LongPolicy<NB, DD, GG, true>;                      \
      using LB = SplitLaunch<PB, 0xA>;                              \
      using LL = SplitLaunch<PL, 0x4>;                              \
      return EXPR;                                                  \
    } else {                                                        \
      using PB = BatchedPolicy<NB, DD, GG, false>;                  \
      using PL = LongPolicy<NB, DD, GG, false>;                     \
      using LB = SplitLaunch<PB, 0xA>;                              \
      using LL = SplitLaunch<PL, 0x4>;                              \
      return EXPR;                                                  \
    }                                                               \
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

static int kchan_unsupported(int nbits, int D, int gs) {
  set_error("fused decode with per-channel keys: unsupported (nbits=%d, head_dim=%d, value "
            "group_size=%d); built: nbits in {2,4}, head_dim in {64,128}, value group_size 32",
            nbits, D, gs);
  return TKV_ERR_UNSUPPORTED;
}

static int fused_unsupported(int nbits, int D, int gs) {
  set_error("fused decode: unsupported (nbits=%d, head_dim=%d, group_size=%d); built: nbits in "
            "{2,4}, head_dim in {64,128}, group_size in {16,32,64,128} with group_size <= head_dim",
            nbits, D, gs);
  return TKV_ERR_UNSUPPORTED;
}

template <class L, class P>
static int fused_launch_one(const DecodeParams& p, const SplitSched& sc, cudaStream_t stream) {
  using C = typename P::C;
  typename P::Maps maps;
  const int64_t rows = (int64_t)p.B * p.HKV * p.S;
  int rc;
  if (p.kv_one) {
    const uint8_t* lo = p.k_second ? p.vp : p.kp;
    const uint8_t* hi = p.k_second ? p.kp : p.vp;
    rc = make_pair_map(&maps.k, lo, (uint64_t)(hi - lo), rows * C::DP / 128, C::kTok * C::DP / 128);
    maps.v = maps.k;
  } else if (p.wide) {
    // [bytes/128, 128] view, box = a tile's bytes as 128-byte rows, 128B swizzle
    rc = make_row_map(&maps.k, p.kp, rows * C::DP / 128, 128, 128, C::kTok * C::DP / 128);
    if (rc != TKV_OK) return rc;
    rc = make_row_map(&maps.v, p.vp, rows * C::DP / 128, 128, 128, C::kTok * C::DP / 128);
  } else {
    rc = make_row_map(&maps.k, p.kp, rows, C::DP, C::DP, C::kTok);
    if (rc != TKV_OK) return rc;
    rc = make_row_map(&maps.v, p.vp, rows, C::DP, C::DP, C::kTok);
  }
  if (rc != TKV_OK) return rc;
  return L::launch(maps, p, sc, stream);
}

// The long family plans first: if its plan is a mode-2 one (unit-aligned, or static units for
// ragged batches with explicit splits) it is taken, otherwise the batched family plans.
template <class LB, class LL>
static int fused_plan_both(SplitSched* sc, int B, int HKV, int hchunks, int S, int num_splits,
                           int split_size, bool ragged) {
  int rc = LL::plan(sc, B, HKV, hchunks, S, num_splits, split_size, ragged);
  if (rc != TKV_OK) return rc;
  if (sc->persistent == 2 || sc->persistent == 0) {
    sc->variant = kVariantLong;
    return TKV_OK;
  }
  rc = LB::plan(sc, B, HKV, hchunks, S, num_splits, split_size, ragged);
  sc->variant = kVariantBatched;
  return rc;
}

int fused_plan(int nbits, int D, int gs, SplitSched* sc, int B, int HKV, int hchunks, int S,
               int num_splits, int split_size, bool ragged, bool kchan) {
  if (kchan) {
    TKV_KCHAN_ALL((fused_plan_both<LB, LL>(sc, B, HKV, hchunks, S, num_splits, split_size, ragged)))
    return kchan_unsupported(nbits, D, gs);
  }
  constexpr bool aligned16_rows = true;  // both instantiations have the same resources
  TKV_FUSED_ALL((fused_plan_both<LB, LL>(sc, B, HKV, hchunks, S, num_splits, split_size, ragged)))
  return fused_unsupported(nbits, D, gs);
}

static int fused_launch(int nbits, int D, int gs, const DecodeParams& p, const SplitSched& sc,
                        cudaStream_t stream, bool kchan) {
  if (kchan) {
    TKV_KCHAN_ALL((sc.variant == kVariantLong ? fused_launch_one<LL, PL>(p, sc, stream)
                                              : fused_launch_one<LB, PB>(p, sc, stream)))
    return kchan_unsupported(nbits, D, gs);
  }
  const bool aligned16_rows = p.meta_aligned == 16;
  TKV_FUSED_ALL((sc.variant == kVariantLong ? fused_launch_one<LL, PL>(p, sc, stream)
                                            : fused_launch_one<LB, PB>(p, sc, stream)))
  return fused_unsupported(nbits, D, gs);
}

// Resources of the batched family (the one that runs where bandwidth binds).
int fused_attrs(int nbits, int D, int gs, int* regs, int* smem, int* local, int* ctas) {
  constexpr bool aligned16_rows = true;
  TKV_FUSED_ALL(LB::attrs(regs, smem, local, ctas))
  return fused_unsupported(nbits, D, gs);
}

int fused_device_status_clear() {
  const int zero = 0;
  TKV_CUDA(cudaMemcpyToSymbol(g_fused_status, &zero, sizeof(int)));
  return TKV_OK;
}

int fused_device_status(int* status) {
  int v = 0;
  TKV_CUDA(cudaMemcpyFromSymbol(&v, g_fused_status, sizeof(int)));
  *status = v;
  return TKV_OK;
}

}  // namespace tkv

extern "C" int tkv_fused_decode(const void* q, int q_dtype, const uint8_t* k_packed,
                                const void* k_scale, const void* k_zero, const uint8_t* v_packed,
                                const void* v_scale, const void* v_zero, float* acc, float* m,
                                float* l, float* out, int B, int HQ, int HKV, int S, int D,
                                int nbits, int gs, float sm_scale, int num_splits, int split_size,
                                int nslots, const int32_t* seq_lens, int flags, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(q && k_packed && k_scale && k_zero && v_packed && v_scale && v_zero, TKV_ERR_INVALID,
              "fused decode: null input pointer");
  DecodeParams p{};
  int rc = fill_common(p, "fused decode", q, q_dtype, acc, m, l, out, B, HQ, HKV, S, sm_scale,
                       num_splits, split_size, nslots, seq_lens, flags);
  if (rc != TKV_OK) return rc;
  TKV_REQUIRE(aligned16(k_packed) && aligned16(v_packed), TKV_ERR_ALIGN,
              "fused decode: packed code pointers must be 16-byte aligned");
  p.kp = k_packed;
  p.vp = v_packed;
  p.ks = (const __half*)k_scale;
  p.kz = (const __half*)k_zero;
  p.vs = (const __half*)v_scale;
  p.vz = (const __half*)v_zero;
  const int ng = (gs > 0 && D % gs == 0) ? D / gs : 0;
  // Alignment of the first byte of any scale/zero tile: the pointers' own alignment, that
  // of a sequence's stride when there is more than one, and 32 bytes inside a sequence
  // (tiles start at multiples of 16 tokens).  The copies use the largest unit that fits.
  {
    const int res = (int)(reinterpret_cast<uintptr_t>(k_scale) & 15);
    TKV_REQUIRE((int)(reinterpret_cast<uintptr_t>(k_zero) & 15) == res &&
                    (int)(reinterpret_cast<uintptr_t>(v_scale) & 15) == res &&
                    (int)(reinterpret_cast<uintptr_t>(v_zero) & 15) == res && (res & 1) == 0,
                TKV_ERR_ALIGN,
                "fused decode: the four scale/zero pointers must share their offset within 16 bytes");
    const int64_t seq_bytes = (int64_t)S * ng * 2;
    const int ptr_al = (res | 16) & -(res | 16);
    const int seq_al = ((int64_t)B * HKV > 1) ? (int)((seq_bytes | 16) & -(seq_bytes | 16)) : 16;
    const int al = ptr_al < seq_al ? ptr_al : seq_al;
    p.meta_aligned = al >= 4 ? al : 0;
    p.meta_phase = res & 3;
    TKV_REQUIRE(al >= 4 || ng == 1, TKV_ERR_ALIGN,
                "fused decode: scale/zero rows of %d bytes must start on 4-byte boundaries", ng * 2);
  }
  // 128-byte-row view of the code tensors: every sequence must start on a 128-byte boundary
  p.wide = (((int64_t)S * D * nbits / 8) % 128 == 0) ? 1 : 0;
  {
    // one tensor map over both code tensors when a tile fills whole 1024-byte swizzle atoms
    const uint8_t* lo = k_packed < v_packed ? k_packed : v_packed;
    const uint8_t* hi = k_packed < v_packed ? v_packed : k_packed;
    const uint64_t gap = (uint64_t)(hi - lo);
    const int64_t tensor_bytes = (int64_t)B * HKV * S * (D * nbits / 8);
    const bool ok = p.wide && ((32 * (D * nbits / 8)) % 1024 == 0) && gap % 16 == 0 && gap < (1ull << 40) &&
                    gap >= (uint64_t)tensor_bytes;
    p.kv_one = ok ? 1 : 0;
    p.k_second = (ok && k_packed > v_packed) ? 1 : 0;
  }
  const bool kchan = (flags & TKV_FLAG_K_PER_CHANNEL) != 0;
  if (kchan) {
    // k_scale / k_zero are (B, HKV, S/32, D): one row per block of 32 tokens, so every tile
    // must be one whole block -- a history of whole blocks, one split, no per-sequence lengths
    TKV_REQUIRE(S % 32 == 0 && num_splits == 1 && seq_lens == nullptr, TKV_ERR_INVALID,
                "fused decode with per-channel keys: S=%d must be a multiple of 32, with one split "
                "and no seq_lens (the fp16 tail goes through tkv_fp16_decode)", S);
    TKV_REQUIRE(aligned16(k_scale) && aligned16(v_scale), TKV_ERR_ALIGN,
                "fused decode with per-channel keys: scale/zero pointers must be 16-byte aligned");
    p.meta_aligned = 16;
  }
  SplitSched sc;
  rc = fused_plan(nbits, D, gs, &sc, B, HKV, p.hchunks, S, num_splits, split_size,
                  seq_lens != nullptr, kchan);
  if (rc != TKV_OK) return rc;
  TKV_REQUIRE(sc.nslots == nslots, TKV_ERR_INVALID,
              "fused decode: nslots=%d does not match the plan (%d); size acc/m/l with "
              "tkv_decode_plan", nslots, sc.nslots);
  rc = fused_launch(nbits, D, gs, p, sc, (cudaStream_t)stream, kchan);
  if (rc != TKV_OK) return rc;
  if ((flags & TKV_FLAG_COMBINE) && nslots > 1 && !(flags & TKV_FLAG_PARTIALS_ONLY)) {
    TKV_REQUIRE(out, TKV_ERR_INVALID, "fused decode: TKV_FLAG_COMBINE needs out");
    return tkv_combine(acc, m, l, out, nullptr, nullptr, B, HQ, nslots, D, stream);
  }
  return TKV_OK;
}
