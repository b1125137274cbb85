// fp16 control: split-K decode attention on an unquantised f16 cache (sm_100a).
//
// Replaces _fp16_decode_attn_split of the reference (kernels/fp16_decode_attn.py:47-135).
// Scheduling, the per-warp copy rings and the epilogue are the shared driver of
// tkv_splitk_driver.cuh -- identical split, online softmax, GQA grouping and partial
// format as the packed-cache kernel; this file is the tile policy: K and V tiles are
// plain f16 rows, fetched with 16-byte cp.async copies into a 128B-swizzled layout
// (completion posted on the stage's mbarrier) and read with ldmatrix (K as the A operand of S^T = K Q^T, V with .trans as
// the A operand of O^T = V^T P^T).
#include "tkv_splitk_driver.cuh"

namespace tkv {

__device__ int g_fp16_status;

template <int D_>
struct Fp16Policy {
  static constexpr int D = D_;
  static constexpr int TOK = 16;
  static constexpr int WARPS = 4;
  static constexpr int STAGES = (D_ >= 128) ? 3 : 4;
  static constexpr int MIN_CTAS = 2;
  static constexpr bool PIPELINED = true;
  static constexpr int BAR_COUNT = 32;  // one arrival per lane
  static constexpr int ROW = 2 * D;            // bytes per token row
  static constexpr int NH = ROW / 128;         // 128-byte column halves per row
  static constexpr int NCH = D / 16;           // 16-dim MMA chunks
  static constexpr int SUB_BYTES = TOK * 128;  // one [16 tokens x 128 bytes] box
  static constexpr int TILE_BYTES = NH * SUB_BYTES;
  static constexpr int PAYLOAD = 2 * TILE_BYTES;
  static constexpr int MERGE_BYTES = kHeadsPerCta * D * 4;
  static constexpr int STAGE_BYTES =
      ((PAYLOAD > MERGE_BYTES ? PAYLOAD : MERGE_BYTES) + 1023) / 1024 * 1024;
  static_assert(ROW % 128 == 0, "head_dim must be a multiple of 64");

  struct Maps {
    int unused;
  };
  struct Query {
    uint32_t qf[NCH][2];
  };
  struct Accum {
    float m_ref0, m_ref1, m_true0, m_true1, l0, l1;
    float acc[NCH][4];
  };

  __device__ static void report_timeout() { atomicExch(&g_fp16_status, 1); }
  __device__ static __forceinline__ void prefetch_maps(const Maps&) {}

  // Byte offset of the 16-byte chunk `c16` (0 .. ROW/16) of token row r inside a tile.
  __device__ static __forceinline__ uint32_t chunk_off(int r, int c16) {
    const int h = c16 >> 3, c = c16 & 7;
    return h * SUB_BYTES + r * 128 + ((c ^ (r & 7)) << 4);
  }


  // Fill one stage with the 16 tokens starting at global row `row`: 16-byte cp.async per
  // lane into the 128B-swizzled layout (rows past the unit end are zero-filled), then one
  // arrival per lane on the stage barrier that fires when the lane's copies have landed.
  struct IssueState {};
  __device__ static __forceinline__ void issue_init(IssueState&, const DecodeParams&, int) {}
  __device__ static __forceinline__ void issue(const IssueState&, const DecodeParams& p,
                                               const Maps& maps, int row, int nvalid, uint32_t st,
                                               uint8_t* st_ptr, uint32_t bar, int lane) {
    constexpr int NCC = TOK * (ROW / 16);  // 16-byte chunks per tile
    const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(p.k) + (int64_t)row * ROW;
    const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(p.v) + (int64_t)row * ROW;
#pragma unroll
    for (int i0 = 0; i0 < NCC; i0 += 32) {
      const int i = i0 + lane;
      const int r = i / (ROW / 16), c16 = i % (ROW / 16);
      const uint32_t dst = chunk_off(r, c16);
      const bool ok = r < nvalid;
      cp_async16(st + dst, ok ? ksrc + i * 16 : reinterpret_cast<const uint8_t*>(p.k), ok ? 16 : 0);
      cp_async16(st + TILE_BYTES + dst, ok ? vsrc + i * 16 : reinterpret_cast<const uint8_t*>(p.v),
                 ok ? 16 : 0);
    }
    cp_async_mbar_arrive_noinc(bar);
  }

  // query fragments: B operand, k-slots (2t,2t+1) <-> dims 16c+2t, 16c+2t+1 and
  // (2t+8, 2t+9) <-> dims 16c+8+2t, 16c+9+2t, column g = head g.
  static constexpr int QFRAG_BYTES = 0;  // every warp reads the query rows itself
  __device__ static __forceinline__ void lane_init(Query&, const DecodeParams&, int) {}
  __device__ static __forceinline__ void build_query(const DecodeParams&, const uint8_t*, uint32_t,
                                                     int, int) {}
  __device__ static __forceinline__ void load_query(Query& qq, const DecodeParams& p,
                                                    const uint8_t* qsm, uint32_t, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* qrow = qsm + g * D * (p.q_dtype == TKV_DTYPE_F32 ? 4 : 2);
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      __half x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = 16 * ch + 2 * t + (i & 1) + (i >> 1) * 8;
        x[i] = load_q_half(qrow, p.q_dtype, d);
      }
      qq.qf[ch][0] = pack_half2(x[0], x[1]);
      qq.qf[ch][1] = pack_half2(x[2], x[3]);
    }
  }

  __device__ static __forceinline__ void reset(Accum& ac) {
    ac.m_ref0 = ac.m_ref1 = ac.m_true0 = ac.m_true1 = -INFINITY;
    ac.l0 = ac.l1 = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
      for (int i = 0; i < 4; ++i) ac.acc[ch][i] = 0.f;
  }

  struct Scores {
    float s[4];  // (token g, head 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
  };

  // Scores of one 16-token tile (scaled, tokens past the unit end set to -inf).
  __device__ static __forceinline__ void scores(Scores& out, const Query& qq, uint32_t st,
                                                const uint8_t* st_ptr, int left, float qk_scale,
                                                int lane) {
    const int g = lane >> 2;
    // K (A operand): matrices (tok 0-7, chunk 2c), (tok 8-15, chunk 2c), (tok 0-7, chunk 2c+1),
    // (tok 8-15, chunk 2c+1)
    const int k_r = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int k_c = lane >> 4;
    float (&sc)[4] = out.s;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      uint32_t r[4];
      ldmatrix_x4(r, st + chunk_off(k_r, 2 * ch + k_c));
      if (ch == 0)
        mma16816_zero(sc, r[0], r[1], r[2], r[3], qq.qf[ch][0], qq.qf[ch][1]);
      else
        mma16816(sc, r[0], r[1], r[2], r[3], qq.qf[ch][0], qq.qf[ch][1]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i] *= qk_scale;
    if (left < TOK) {
      if (g >= left) sc[0] = sc[1] = -INFINITY;
      if (g + 8 >= left) sc[2] = sc[3] = -INFINITY;
    }
  }

  // Online softmax update and O^T += V^T P^T for the tile whose scores are `in`.
  __device__ static __forceinline__ void update(Accum& ac, const Query& qq, Scores& in,
                                                uint32_t st, uint8_t* st_ptr, int left, int lane) {
    const uint32_t vt = st + TILE_BYTES;
    float (&sc)[4] = in.s;
    // V (A operand of O^T, via .trans): matrices (tok 0-7, chunk 2i), (tok 0-7, chunk 2i+1),
    // (tok 8-15, chunk 2i), (tok 8-15, chunk 2i+1)
    const int v_r = (lane & 7) + (lane >> 4) * 8;
    const int v_c = (lane >> 3) & 1;

    // online softmax with a lazily raised reference exponent
    {
      float mx0 = fmaxf(sc[0], sc[2]);
      float mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
      for (int off = 4; off <= 16; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, off));
      }
      ac.m_true0 = fmaxf(ac.m_true0, mx0);
      ac.m_true1 = fmaxf(ac.m_true1, mx1);
      if (__any_sync(kFullMask, (mx0 > ac.m_ref0) || (mx1 > ac.m_ref1))) {
        const float n0 = (mx0 > ac.m_ref0) ? mx0 + kLazyTau : ac.m_ref0;
        const float n1 = (mx1 > ac.m_ref1) ? mx1 + kLazyTau : ac.m_ref1;
        const float alpha0 = ex2(ac.m_ref0 - n0);
        const float alpha1 = ex2(ac.m_ref1 - n1);
        ac.m_ref0 = n0;
        ac.m_ref1 = n1;
        ac.l0 *= alpha0;
        ac.l1 *= alpha1;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          ac.acc[ch][0] *= alpha0;
          ac.acc[ch][1] *= alpha1;
          ac.acc[ch][2] *= alpha0;
          ac.acc[ch][3] *= alpha1;
        }
      }
      sc[0] = ex2(sc[0] - ac.m_ref0);
      sc[1] = ex2(sc[1] - ac.m_ref1);
      sc[2] = ex2(sc[2] - ac.m_ref0);
      sc[3] = ex2(sc[3] - ac.m_ref1);
      ac.l0 += sc[0] + sc[2];
      ac.l1 += sc[1] + sc[3];
    }

    const uint32_t pb0 = movmatrix_trans(pack_half2(sc[0], sc[1]));
    const uint32_t pb1 = movmatrix_trans(pack_half2(sc[2], sc[3]));
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      uint32_t r[4];
      ldmatrix_x4_trans(r, vt + chunk_off(v_r, 2 * ch + v_c));
      mma16816(ac.acc[ch], r[0], r[1], r[2], r[3], pb0, pb1);
    }
  }

  __device__ static __forceinline__ void finalize(Accum& ac, float* vals, SoftmaxState& st,
                                                  int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
      ac.l0 += __shfl_xor_sync(kFullMask, ac.l0, off);
      ac.l1 += __shfl_xor_sync(kFullMask, ac.l1, off);
    }
    const float f0 = (ac.m_true0 == -INFINITY) ? 0.f : ex2(ac.m_ref0 - ac.m_true0);
    const float f1 = (ac.m_true1 == -INFINITY) ? 0.f : ex2(ac.m_ref1 - ac.m_true1);
    st = SoftmaxState{ac.m_true0, ac.m_true1, ac.l0 * f0, ac.l1 * f1};
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      // rows g / g+8 of output tile ch are dims 16ch+g / 16ch+8+g; columns heads 2t, 2t+1
      vals[(2 * t) * D + 16 * ch + g] = ac.acc[ch][0] * f0;
      vals[(2 * t + 1) * D + 16 * ch + g] = ac.acc[ch][1] * f1;
      vals[(2 * t) * D + 16 * ch + 8 + g] = ac.acc[ch][2] * f0;
      vals[(2 * t + 1) * D + 16 * ch + 8 + g] = ac.acc[ch][3] * f1;
    }
  }
};

static int fp16_unsupported(int D) {
  set_error("fp16 decode: unsupported head_dim=%d (built: 64, 128)", D);
  return TKV_ERR_UNSUPPORTED;
}

int fp16_plan(int D, SplitSched* sc, int B, int HKV, int hchunks, int S, int num_splits,
              int split_size, bool ragged) {
  if (D == 128)
    return SplitLaunch<Fp16Policy<128>>::plan(sc, B, HKV, hchunks, S, num_splits, split_size, ragged);
  if (D == 64)
    return SplitLaunch<Fp16Policy<64>>::plan(sc, B, HKV, hchunks, S, num_splits, split_size, ragged);
  return fp16_unsupported(D);
}

int fp16_attrs(int D, int* regs, int* smem, int* local, int* ctas) {
  if (D == 128) return SplitLaunch<Fp16Policy<128>>::attrs(regs, smem, local, ctas);
  if (D == 64) return SplitLaunch<Fp16Policy<64>>::attrs(regs, smem, local, ctas);
  return fp16_unsupported(D);
}

int fp16_device_status_clear() {
  const int zero = 0;
  TKV_CUDA(cudaMemcpyToSymbol(g_fp16_status, &zero, sizeof(int)));
  return TKV_OK;
}

int fp16_device_status(int* status) {
  int v = 0;
  TKV_CUDA(cudaMemcpyFromSymbol(&v, g_fp16_status, sizeof(int)));
  *status = v;
  return TKV_OK;
}

template <int D>
static int fp16_launch_one(const DecodeParams& p, const SplitSched& sc, cudaStream_t stream) {
  using P = Fp16Policy<D>;
  typename P::Maps maps;
  const int64_t rows = (int64_t)p.B * p.HKV * p.S;
  (void)rows;  // the control kernel addresses K and V directly; no tensor maps
  maps.unused = 0;
  return SplitLaunch<P>::launch(maps, p, sc, stream);
}

}  // namespace tkv

extern "C" int tkv_fp16_decode(const void* q, int q_dtype, const void* k, const void* v, float* acc,
                               float* m, float* l, float* out, int B, int HQ, int HKV, int S, int D,
                               float sm_scale, int num_splits, int split_size, int nslots,
                               const int32_t* seq_lens, int flags, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(q && k && v, TKV_ERR_INVALID, "fp16 decode: null input pointer");
  DecodeParams p{};
  int rc = fill_common(p, "fp16 decode", q, q_dtype, acc, m, l, out, B, HQ, HKV, S, sm_scale,
                       num_splits, split_size, nslots, seq_lens, flags);
  if (rc != TKV_OK) return rc;
  TKV_REQUIRE(aligned16(k) && aligned16(v), TKV_ERR_ALIGN,
              "fp16 decode: k and v pointers must be 16-byte aligned");
  p.k = (const __half*)k;
  p.v = (const __half*)v;
  SplitSched sc;
  rc = fp16_plan(D, &sc, B, HKV, p.hchunks, S, num_splits, split_size, seq_lens != nullptr);
  if (rc != TKV_OK) return rc;
  TKV_REQUIRE(sc.nslots == nslots, TKV_ERR_INVALID,
              "fp16 decode: nslots=%d does not match the plan (%d); size acc/m/l with "
              "tkv_decode_plan", nslots, sc.nslots);
  if (D == 128) rc = fp16_launch_one<128>(p, sc, (cudaStream_t)stream);
  else if (D == 64) rc = fp16_launch_one<64>(p, sc, (cudaStream_t)stream);
  else return fp16_unsupported(D);
  if (rc != TKV_OK) return rc;
  if ((flags & TKV_FLAG_COMBINE) && nslots > 1 && !(flags & TKV_FLAG_PARTIALS_ONLY)) {
    TKV_REQUIRE(out, TKV_ERR_INVALID, "fp16 decode: TKV_FLAG_COMBINE needs out");
    return tkv_combine(acc, m, l, out, nullptr, nullptr, B, HQ, nslots, D, stream);
  }
  return TKV_OK;
}
