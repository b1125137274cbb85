// Persistent, balanced split-K driver shared by the packed-cache kernel and the fp16
// control kernel (sm_100a).
//
// Work model.  A "unit" is one (batch, KV head, head chunk, history split); its tokens
// are cut into tiles of Policy::TOK tokens.  All tiles of all units form one global sequence.  The
// grid is one wave of persistent CTAs; CTA c owns the contiguous global tile range
// [c*TC, (c+1)*TC).  Where that range crosses unit boundaries the CTA processes one
// "segment" per unit and emits one partial (acc, m, l) per segment, so every CTA does
// the same number of tiles (+-1) whatever the batch and history sizes are -- no ragged
// last wave, no per-unit launch cost -- and the reference's split geometry
// (kernels/fused_decode_attn.py:493-499) survives as the unit boundaries.
// Partial slot of a segment: split*SEG + (c - first CTA touching the unit); the CTA
// that finishes a unit marks the unit's unused slots empty (m = -inf).
//
// Inside a CTA every warp is an independent stream with a private ring of STAGES
// shared-memory stages and one mbarrier per stage.  Lane 0 issues the copies of a
// tile (Policy::issue); the ring keeps running across segment boundaries, so the next
// unit's first tiles are already in flight while a segment's epilogue runs.  The tile
// loop has two forms (Policy::PIPELINED): a software pipeline that holds two tiles per
// warp (scores of tile i+1 beside the update of tile i; needs STAGES >= 3), and a
// one-tile-at-a-time form whose body exists once per ring slot (STAGES >= 2), which
// fits more warps per SM in the same shared memory.  Warps
// only meet at a segment end: each writes its partial into its one free stage, the
// CTA merges the warps' partials (log-sum-exp) and stores the segment's partial or,
// when a unit has a single slot, the normalised output.
//
// With per-sequence lengths (seq_lens) the schedule is static instead: CTA c <-> unit c.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "tkv_split_common.cuh"

namespace tkv {

constexpr int kMaxRaggedB = 512;  // sequences whose tile prefix fits the kernel's static shared memory
constexpr float kLazyTau = 4.0f;  // head-room of the lazily raised softmax exponent (log2 units)

// n / d for 0 <= n < 2^31 and a divisor fixed per launch, as a multiply-high, an add and a
// shift: the pair is made on the host.  (A 32-bit division is ~40 instructions, a 64-bit one
// several hundred cycles; a segment look-up has five and every warp performs it.)
struct FastDiv {
  uint32_t mul, shift;
};
inline FastDiv make_fastdiv(int d) {
  const uint64_t dd = d > 1 ? (uint64_t)d : 1;
  uint32_t l = 0;
  while ((1ull << l) < dd) ++l;
  FastDiv f;
  f.mul = (uint32_t)(((1ull << 32) * ((1ull << l) - dd)) / dd + 1);
  f.shift = l;
  return f;
}
__device__ __forceinline__ FastDiv make_fastdiv_device(int d) {  // one 64-bit division, once per CTA
  const uint32_t dd = d > 1 ? (uint32_t)d : 1u;
  const uint32_t l = dd > 1 ? 32u - (uint32_t)__clz((int)(dd - 1)) : 0u;
  FastDiv f;
  f.mul = (uint32_t)(((1ull << 32) * ((1ull << l) - dd)) / dd + 1);
  f.shift = l;
  return f;
}
__device__ __forceinline__ int fast_div(int n, FastDiv f) {
  return (int)((__umulhi((uint32_t)n, f.mul) + (uint32_t)n) >> f.shift);
}

struct SplitSched {
  int persistent;  // 0: CTA c <-> unit c (ragged batches with explicit splits); 1: balanced
                   // tile ranges over the global tile sequence; 2: SEG CTAs per unit, ranges
                   // aligned to the unit; 3: balanced ranges over a ragged batch, the tile
                   // sequence built on the device from seq_lens
  int NS;          // history splits per sequence (unit boundaries)
  int TUf, TUl;    // tiles in a full split / in the last split
  int T_seq;       // tiles per sequence = (NS-1)*TUf + TUl
  int T;           // total tiles
  int TC;          // tiles per CTA
  int SEG;         // partial slots per split
  int nslots;      // NS * SEG
  int grid;        // CTAs
  int HKVc;        // HKV * head chunks
  int variant;     // which kernel instantiation the plan was made for (set by the planner)
  FastDiv dSEG, dNS, dHKVc, dTseq, dTUf, dTC, dHch;  // divisions by SEG, NS, HKVc, T_seq, TUf, TC, head chunks
};

// `unit_aligned`: whether the plan may be the unit-aligned one (mode 2); a kernel family that
// is only built for the balanced modes passes false.
inline SplitSched make_sched(int B, int HKV, int hchunks, int S, int num_splits, int split_size,
                             bool ragged, int wave, int kTok, int warps, bool unit_aligned = true) {
  SplitSched s{};
  s.NS = num_splits;
  s.HKVc = HKV * hchunks;
  const int last_len = S - (num_splits - 1) * split_size;
  s.TUf = (num_splits > 1 ? split_size : S) > 0 ? ((num_splits > 1 ? split_size : S) + kTok - 1) / kTok : 0;
  s.TUl = (last_len + kTok - 1) / kTok;
  if (num_splits == 1) s.TUf = s.TUl;
  s.T_seq = (num_splits - 1) * s.TUf + s.TUl;
  const int64_t units = (int64_t)B * s.HKVc * num_splits;
  if (ragged && num_splits == 1 && B <= kMaxRaggedB && (int64_t)B * s.TUf < (1 << 25)) {  // (prefix words hold 25 bits of tiles)
    // Lengths live on the device, so only bounds are known here: one wave of CTAs, and
    // per unit at most min(tiles, wave/HKVc + 2) segments (a unit of t tiles is cut into
    // at most t/TC + 2 ranges and TC >= HKVc * t / wave).
    s.persistent = 3;
    s.T = 0;
    s.TC = 0;
    s.grid = wave;
    const int by_wave = wave / s.HKVc + 2;
    s.SEG = s.TUf < by_wave ? s.TUf : by_wave;
    if (s.SEG < 1) s.SEG = 1;
  } else if (ragged) {
    s.persistent = 0;
    s.T = 0;
    s.TC = 0;
    s.SEG = 1;
    s.grid = (int)units;
  } else {
    s.persistent = 1;
    const int64_t T = (int64_t)B * s.HKVc * s.T_seq;
    s.T = (int)T;
    const int G = (int)(T < wave ? T : wave);
    s.TC = (int)((T + G - 1) / G);
    s.grid = (int)((T + s.TC - 1) / s.TC);
    s.SEG = (s.TUf - 1 + s.TC - 1) / s.TC + 1;
    if (s.TUf <= 1) s.SEG = 1;
    // Few, long units (small batches): give every unit its own whole number of CTAs, so
    // that no CTA straddles two units and pays a second query load and epilogue.  Taken
    // when it lengthens the longest CTA by at most one tile.
    // CTA j of a unit's SEG takes tiles [j*TU/SEG, (j+1)*TU/SEG): every resident slot of
    // the device is used and tile counts differ by at most one.
    if (unit_aligned && units * 2 <= wave) {
      const int cpu = (int)(wave / units);
      // no more CTAs per unit than give every warp of a CTA a tile: spreading a short
      // history thinner only adds partials for the combine to read
      const int by_warps = (s.TUf + warps - 1) / warps;
      const int SEGu = by_warps < cpu ? by_warps : cpu;
      const int TCu = (s.TUf + SEGu - 1) / SEGu;
      if (TCu <= s.TC + 1 || TCu <= warps) {
        s.persistent = 2;
        s.TC = TCu;
        s.SEG = SEGu;
        s.grid = (int)(units * s.SEG);
      }
    }
  }
  s.nslots = s.NS * s.SEG;
  s.dSEG = make_fastdiv(s.SEG);
  s.dNS = make_fastdiv(s.NS);
  s.dHKVc = make_fastdiv(s.HKVc);
  s.dTseq = make_fastdiv(s.T_seq);
  s.dTUf = make_fastdiv(s.TUf);
  s.dTC = make_fastdiv(s.TC);
  s.dHch = make_fastdiv(hchunks);
  return s;
}

// One segment: the part of one unit that one CTA processes.
struct Segment {
  int b, hkv, hc;     // unit coordinates
  int split;          // history split index
  int lo_tok;         // first token of the segment (absolute, within the sequence)
  int hi;             // end of the unit's token range (exclusive)
  int ntiles;         // tiles in this segment
  int g_end;          // global tile index one past the segment (persistent mode)
  int slot;           // partial slot
  int fill_from;      // if >= 0: after the epilogue mark slots [fill_from, fill_to) empty
  int fill_to;
};

template <int kTok>
__device__ __forceinline__ Segment segment_at(const DecodeParams& p, const SplitSched& sc, int g,
                                              int g1, int cta) {
  Segment s;
  const int bh = fast_div(g, sc.dTseq);
  const int r = g - bh * sc.T_seq;
  const int sp = min(fast_div(r, sc.dTUf), sc.NS - 1);
  const int tu = r - sp * sc.TUf;
  const int TU = (sp == sc.NS - 1) ? sc.TUl : sc.TUf;
  const int unit_start = bh * sc.T_seq + sp * sc.TUf;
  const int unit_end = unit_start + TU;
  s.b = fast_div(bh, sc.dHKVc);
  const int hk = bh - s.b * sc.HKVc;
  s.hkv = fast_div(hk, sc.dHch);
  s.hc = hk - s.hkv * p.hchunks;
  s.split = sp;
  const int lo_unit = sp * p.split_size;
  s.hi = min(lo_unit + p.split_size, p.S);
  s.lo_tok = lo_unit + tu * kTok;
  s.g_end = min(g1, unit_end);
  s.ntiles = s.g_end - g;
  const int c_first = fast_div(unit_start, sc.dTC);
  const int seg = cta - c_first;
  s.slot = sp * sc.SEG + seg;
  if (s.g_end == unit_end && seg + 1 < sc.SEG) {
    s.fill_from = s.slot + 1;
    s.fill_to = sp * sc.SEG + sc.SEG;
  } else {
    s.fill_from = -1;
    s.fill_to = -1;
  }
  return s;
}

// Ragged batches: `pref[b]` = tiles of sequences 0..b-1 (one KV head), so unit
// (b, hk) starts at global tile HKVc*pref[b] + hk*t_b with t_b = pref[b+1] - pref[b].
// An entry of `pref` is (tiles before the sequence) << kRemBits | (tokens in its last tile - 1),
// so a sequence's length comes out of the same words as its tile range; `dTC` divides by the
// tiles per CTA.
constexpr int kRemBits = 6;  // a tile has at most 64 tokens
template <int kTok>
__device__ __forceinline__ Segment ragged_segment_at(const DecodeParams& p, const SplitSched& sc,
                                                     const int* pref, FastDiv dTC, int g, int g1,
                                                     int cta) {
  static_assert(kTok <= (1 << kRemBits), "the remainder field holds tokens of one tile");
  Segment s;
  int lo = 0, hi = p.B;  // largest b with HKVc*pref[b] <= g (sequences without tiles are skipped)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sc.HKVc * (pref[mid] >> kRemBits) <= g) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int word = pref[b], before = word >> kRemBits;
  const int t_b = (pref[b + 1] >> kRemBits) - before;
  const int r = g - sc.HKVc * before;
  const int hk = (int)((uint32_t)r / (uint32_t)t_b);  // (unsigned: half the instructions of a signed division)
  const int tile = r - hk * t_b;
  const int unit_start = g - tile, unit_end = unit_start + t_b;
  s.b = b;
  s.hkv = fast_div(hk, sc.dHch);
  s.hc = hk - s.hkv * p.hchunks;
  s.split = 0;
  s.hi = (t_b - 1) * kTok + (word & ((1 << kRemBits) - 1)) + 1;  // the length, clamped to [1, S] (t_b >= 1 here)
  s.lo_tok = tile * kTok;
  s.g_end = min(g1, unit_end);
  s.ntiles = s.g_end - g;
  const int seg = cta - fast_div(unit_start, dTC);
  s.slot = seg;
  if (s.g_end == unit_end && seg + 1 < sc.SEG) {
    s.fill_from = seg + 1;
    s.fill_to = sc.SEG;
  } else {
    s.fill_from = -1;
    s.fill_to = -1;
  }
  return s;
}

// Per-warp cursor over the tiles this warp will issue, possibly segments ahead.
struct IssueCursor {
  int seg_g;      // global tile index where the cursor's segment starts (persistent mode)
  int row;        // global row (token index over the whole cache tensor, < 2^31) of the next tile
  int left;       // tokens from the next tile's first token to the end of its unit
  int cnt;        // tiles this warp still has to issue in the cursor's segment
  int g_end;      // end of the cursor's segment
};

// MODE: 1 = balanced ranges over the dense tile sequence, 3 = the same over a ragged batch,
// 2 = one segment per CTA (unit-aligned plans and the static plan).  A compile-time mode
// keeps the single-segment kernel -- the latency-critical one, small batches -- free of the
// segment look-ups, which are inlined at seven places in the others.
template <class Policy, int MODE>
__global__ void __launch_bounds__(Policy::WARPS * 32, Policy::MIN_CTAS)
    splitk_kernel(const __grid_constant__ typename Policy::Maps maps, const DecodeParams p,
                  const SplitSched sc) {
  constexpr int WARPS = Policy::WARPS, STAGES = Policy::STAGES, D = Policy::D;
  constexpr int kTok = Policy::TOK;
  constexpr int kLog2D = D == 64 ? 6 : (D == 128 ? 7 : (D == 256 ? 8 : 5));
  static_assert((1 << kLog2D) == D, "head_dim is a power of two between 32 and 256");
  constexpr int STAGE_BYTES = Policy::STAGE_BYTES;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep 1024-byte alignment");
  static_assert(STAGES >= (Policy::PIPELINED ? 3 : 2),
                "pipelined: two tiles resident and one in flight; else one resident, one in flight");
  static_assert(Policy::PIPELINED || STAGES <= 3,
                "the per-slot tile bodies are written for rings of 2 or 3 stages");
  static_assert(STAGE_BYTES >= kHeadsPerCta * D * 4, "a stage must hold one warp's partial");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  __shared__ float s_m[WARPS][kHeadsPerCta];
  __shared__ float s_l[WARPS][kHeadsPerCta];
  __shared__ int s_slot[WARPS];

  // the shuffle tells the compiler that the warp index is warp-uniform, so the ring, cursor and
  // barrier arithmetic that hangs off it can go to the uniform datapath
  const int warp = __shfl_sync(kFullMask, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  // The whole grid is resident at once, so the combine kernel that follows may be
  // scheduled right away; it waits for this grid's completion before it reads anything.
  pdl_launch_dependents();
  if (threadIdx.x == 0) Policy::prefetch_maps(maps);

  uint8_t* ring = smem + (size_t)warp * STAGES * STAGE_BYTES;
  const uint32_t ring_u32 = smem_u32(ring);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)WARPS * STAGES * STAGE_BYTES);
  const uint32_t bar_u32 = smem_u32(bars + warp * STAGES);
  // query rows of a segment (8 heads x D, raw dtype) are staged in shared memory and
  // prefetched one segment ahead: a global load issued when it is needed waits behind the
  // whole copy stream (measured ~3 us under load), which the prefetch hides.
  constexpr int QB = kHeadsPerCta * D * 4;
  uint64_t* qbars = bars + WARPS * STAGES;
  const uint32_t qbar_u32 = smem_u32(qbars);
  uint8_t* qbuf = reinterpret_cast<uint8_t*>(qbars + 2);
  const uint32_t qbuf_u32 = smem_u32(qbuf);
  const uint32_t qfrag_u32 = qbuf_u32 + 2 * QB;  // query fragments shared by the warps
  // ragged batches only (the launch adds the bytes): tiles before each sequence
  int* s_pref = reinterpret_cast<int*>(qbuf + 2 * QB + ((Policy::QFRAG_BYTES + 15) & ~15));
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + 8 * s, Policy::BAR_COUNT);
    if (warp == 0) {
      mbar_init(qbar_u32, WARPS * 32);
      mbar_init(qbar_u32 + 8, WARPS * 32);
    }
    fence_barrier_init();
  }
  const int q_esz = p.q_dtype == TKV_DTYPE_F32 ? 4 : 2;
  auto prefetch_q = [&](int slot, int b, int hkv, int hc) {
    const int row_bytes = D * q_esz, cpr = row_bytes >> 4, cpr_shift = q_esz == 4 ? kLog2D - 2 : kLog2D - 3;
    for (int i = threadIdx.x; i < kHeadsPerCta * cpr; i += WARPS * 32) {
      const int h = i >> cpr_shift, c = i - (h << cpr_shift);
      const int hg = hc * kHeadsPerCta + h;
      const bool ok = hg < p.group;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q) +
                           (((int64_t)b * p.HQ + (int64_t)hkv * p.group + hg) * D) * q_esz + c * 16;
      cp_async16(qbuf_u32 + slot * QB + h * row_bytes + c * 16,
                 ok ? src : reinterpret_cast<const uint8_t*>(p.q), ok ? 16 : 0);
    }
    cp_async_mbar_arrive_noinc(qbar_u32 + 8 * slot);
  };

  // ---- this CTA's tile range ----
  int g0, g1;
  int TC = sc.TC;  // tiles per CTA (computed here for ragged batches)
  FastDiv dTC = sc.dTC;
  Segment seg;
  constexpr bool kMulti = (MODE & 1) != 0;  // a CTA may serve several segments
  auto seg_at = [&](int g, int g_hi) {
    if constexpr (MODE == 3) {
      return ragged_segment_at<kTok>(p, sc, s_pref, dTC, g, g_hi, cta);
    } else if constexpr (MODE == 1) {
      return segment_at<kTok>(p, sc, g, g_hi, cta);
    } else {
      (void)g;
      (void)g_hi;
      return Segment{};
    }
  };
  if constexpr (MODE == 1) {
    g0 = min(cta * sc.TC, sc.T);
    g1 = min(g0 + sc.TC, sc.T);
    if (g0 >= g1) return;
    seg = segment_at<kTok>(p, sc, g0, g1, cta);
  } else if constexpr (MODE == 3) {
    // balanced ranges over a ragged batch: every CTA builds the tile prefix of the
    // sequences (warp 0, 32 at a time), then cuts the global tile sequence evenly
    pdl_wait();
    if (warp == 0) {
      int carry = 0;
      for (int b0 = 0; b0 < p.B; b0 += 32) {
        const int b = b0 + lane;
        const int len = b < p.B ? min(max(p.seq_lens[b], 0), p.S) : 0;
        int t = (len + kTok - 1) / kTok, incl = t;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int y = __shfl_up_sync(kFullMask, incl, off);
          if (lane >= off) incl += y;
        }
        if (b < p.B)
          s_pref[b] = ((carry + incl - t) << kRemBits) | (t > 0 ? len - (t - 1) * kTok - 1 : 0);
        carry += __shfl_sync(kFullMask, incl, 31);
      }
      if (lane == 0) s_pref[p.B] = carry << kRemBits;
    }
    __syncthreads();
    const int T = sc.HKVc * (s_pref[p.B] >> kRemBits);
    TC = max(1, (T + (int)gridDim.x - 1) / (int)gridDim.x);
    dTC = make_fastdiv_device(TC);
    // units without tokens are touched by no range: their slots are marked empty here
    for (int u = cta; u < p.B * sc.HKVc; u += gridDim.x) {
      const int b = u / sc.HKVc, hk = u - b * sc.HKVc;
      const bool no_tiles = (s_pref[b + 1] >> kRemBits) == (s_pref[b] >> kRemBits);
      if (no_tiles && p.partials) {
        const int hkv = hk / p.hchunks, hc = hk - hkv * p.hchunks;
        for (int idx = threadIdx.x; idx < kHeadsPerCta * sc.SEG; idx += WARPS * 32) {
          const int h = idx / sc.SEG, j = idx - h * sc.SEG;
          const int hg = hc * kHeadsPerCta + h;
          if (hg < p.group) {
            const int64_t hq = (int64_t)b * p.HQ + hkv * p.group + hg;
            p.m[hq * sc.nslots + j] = -INFINITY;
            p.l[hq * sc.nslots + j] = 0.f;
          }
        }
      } else if (no_tiles) {
        for (int idx = threadIdx.x; idx < kHeadsPerCta * D; idx += WARPS * 32) {
          const int h = idx / D, d = idx - h * D;
          const int hkv = hk / p.hchunks, hc = hk - hkv * p.hchunks;
          const int hg = hc * kHeadsPerCta + h;
          if (hg < p.group) p.out[((int64_t)b * p.HQ + hkv * p.group + hg) * D + d] = 0.f;
        }
      }
    }
    g0 = min(cta * TC, T);
    g1 = min(g0 + TC, T);
    if (g0 >= g1) return;
    seg = seg_at(g0, g1);
  } else if (sc.persistent == 2) {  // MODE 2 from here on
    // unit-aligned: CTA j of the unit's SEG takes tiles [j*TU/SEG, (j+1)*TU/SEG) of the unit
    const int u = fast_div(cta, sc.dSEG), j = cta - u * sc.SEG;
    const int bh = fast_div(u, sc.dNS);
    seg.split = u - bh * sc.NS;
    seg.b = fast_div(bh, sc.dHKVc);
    const int hk = bh - seg.b * sc.HKVc;
    seg.hkv = fast_div(hk, sc.dHch);
    seg.hc = hk - seg.hkv * p.hchunks;
    const int TU = (seg.split == sc.NS - 1) ? sc.TUl : sc.TUf;
    // floor(j*TU/SEG) = j*(TU/SEG) + floor(j*(TU%SEG)/SEG): all products stay below SEG^2
    const int tq = fast_div(TU, sc.dSEG), tr = TU - tq * sc.SEG;
    const int t0 = j * tq + fast_div(j * tr, sc.dSEG);
    const int lo_unit = seg.split * p.split_size;
    seg.hi = min(lo_unit + p.split_size, p.S);
    seg.lo_tok = lo_unit + t0 * kTok;
    seg.ntiles = (j + 1) * tq + fast_div((j + 1) * tr, sc.dSEG) - t0;
    seg.slot = seg.split * sc.SEG + j;
    seg.fill_from = seg.fill_to = -1;
    g0 = 0;
    g1 = seg.ntiles;
    seg.g_end = g1;
    if (seg.ntiles <= 0) {
      // a shorter last split leaves this CTA without tiles: its slot is marked empty
      pdl_wait();
      if (threadIdx.x < kHeadsPerCta) {
        const int hg = seg.hc * kHeadsPerCta + threadIdx.x;
        if (hg < p.group) {
          const int64_t hq = (int64_t)seg.b * p.HQ + seg.hkv * p.group + hg;
          p.m[hq * sc.nslots + seg.slot] = -INFINITY;
          p.l[hq * sc.nslots + seg.slot] = 0.f;
        }
      }
      return;
    }
  } else {
    // static: CTA <-> unit, per-sequence length from seq_lens
    pdl_wait();
    const int bh = fast_div(cta, sc.dNS);
    seg.split = cta - bh * sc.NS;
    seg.b = fast_div(bh, sc.dHKVc);
    const int hk = bh - seg.b * sc.HKVc;
    seg.hkv = fast_div(hk, sc.dHch);
    seg.hc = hk - seg.hkv * p.hchunks;
    const int S_b = p.seq_lens ? min(max(p.seq_lens[seg.b], 0), p.S) : p.S;
    const int lo_unit = seg.split * p.split_size;
    seg.hi = min(lo_unit + p.split_size, S_b);
    seg.lo_tok = lo_unit;
    seg.ntiles = seg.hi > lo_unit ? (seg.hi - lo_unit + kTok - 1) / kTok : 0;
    seg.slot = seg.split;
    seg.fill_from = seg.fill_to = -1;
    g0 = 0;
    g1 = seg.ntiles;
    seg.g_end = g1;
  }

  __syncthreads();  // barriers initialised

  // ---- issue cursor ----
  auto cursor_enter = [&](IssueCursor& c, const Segment& s, int seg_g) {
    c.seg_g = seg_g;
    c.g_end = s.g_end;
    c.cnt = s.ntiles > warp ? (s.ntiles - warp + WARPS - 1) / WARPS : 0;
    const int tok = s.lo_tok + warp * kTok;
    c.row = (s.b * p.HKV + s.hkv) * p.S + tok;
    c.left = s.hi - tok;
  };
  typename Policy::IssueState ist;
  Policy::issue_init(ist, p, lane);
  IssueCursor cur;
  cursor_enter(cur, seg, g0);
  auto cursor_skip_empty = [&]() {
    // move to the next segment in which this warp has a tile (persistent mode only)
    if constexpr (kMulti) {
      while (cur.cnt == 0 && cur.g_end < g1) {
        const int g = cur.g_end;
        const Segment s = seg_at(g, g1);
        cursor_enter(cur, s, g);
      }
    }
  };
  cursor_skip_empty();
  // Ring positions are kept as (slot, phase) and stepped with a compare, not derived
  // from running counters: STAGES is 3, and a modulo per use was tens of instructions
  // per tile.
  int iss_slot = 0;  // slot the next issue fills
  bool need_proxy_fence = false;
  auto issue_at = [&](int slot) {
    if (cur.cnt == 0) return;
    iss_slot = (slot + 1 == STAGES) ? 0 : slot + 1;
    if (need_proxy_fence) {  // a generic-proxy epilogue touched the ring since the last issue
      fence_proxy_async();
      need_proxy_fence = false;
    }
    Policy::issue(ist, p, maps, cur.row, min(kTok, cur.left), ring_u32 + slot * STAGE_BYTES,
                  ring + slot * STAGE_BYTES, bar_u32 + 8 * slot, lane);
    cur.row += WARPS * kTok;
    cur.left -= WARPS * kTok;
    --cur.cnt;
    cursor_skip_empty();
  };
  auto issue_next = [&]() { issue_at(iss_slot); };
  typename Policy::Query qs;
  Policy::lane_init(qs, p, lane);
  // Launched as a programmatic dependent: everything above ran while the previous kernel
  // of the stream was finishing; global memory is touched only from here on.
  pdl_wait();
  // The query rows go first: behind the first tiles of every warp of the grid they would
  // queue for microseconds, ahead of them they arrive while the tiles are being issued.
  prefetch_q(0, seg.b, seg.hkv, seg.hc);
#pragma unroll 1  // one copy of the issue code here: a cold instruction cache pays per byte
  for (int s = 0; s < (Policy::PIPELINED ? STAGES - 1 : STAGES); ++s) issue_next();
  if constexpr (kMulti) {
    if (seg.g_end < g1) {
      const Segment s1 = seg_at(seg.g_end, g1);
      prefetch_q(1, s1.b, s1.hkv, s1.hc);
    }
  }
  int seg_k = 0;  // index of the current segment within this CTA

  int c_slot = 0, c_phase = 0;  // slot and barrier phase of the next tile to consume
  bool timed_out = false;
  bool deferred_issue = false;  // one-tile form: the refill of the stage that carries the partial
  typename Policy::Accum acc;

  for (int g = g0;;) {
    // ---- one segment ----
    if (!mbar_wait_bounded(qbar_u32 + 8 * (seg_k & 1), (seg_k >> 1) & 1)) timed_out = true;
    if (Policy::QFRAG_BYTES > 0) {
      Policy::build_query(p, qbuf + (seg_k & 1) * QB, qfrag_u32, warp, lane);
      __syncthreads();
    }
    Policy::load_query(qs, p, qbuf + (seg_k & 1) * QB, qfrag_u32, lane);
    Policy::reset(acc);
    const int my_tiles = seg.ntiles > warp ? (seg.ntiles - warp + WARPS - 1) / WARPS : 0;
    int left = seg.hi - (seg.lo_tok + warp * kTok);
    if constexpr (Policy::PIPELINED) {
      // Software pipeline: the scores of tile i+1 are computed in the same straight-line
      // block as the softmax/output update of tile i, so the two independent dependency
      // chains interleave in the instruction stream.
      if (my_tiles > 0 && !timed_out) {
        typename Policy::Scores sc_cur;
        if (!mbar_wait_bounded(bar_u32 + 8 * c_slot, c_phase)) timed_out = true;
        __syncwarp();
        if (!timed_out)
          Policy::scores(sc_cur, qs, ring_u32 + c_slot * STAGE_BYTES, ring + c_slot * STAGE_BYTES, left,
                         p.qk_scale, lane);
        for (int i = 1; i < my_tiles && !timed_out; ++i) {
          int n_slot = c_slot + 1, n_phase = c_phase;
          if (n_slot == STAGES) {
            n_slot = 0;
            n_phase ^= 1;
          }
          if (!mbar_wait_bounded(bar_u32 + 8 * n_slot, n_phase)) {
            timed_out = true;
            break;
          }
          __syncwarp();
          issue_next();  // refills the stage whose tile was finished in the previous iteration
          typename Policy::Scores sc_next;
          Policy::scores(sc_next, qs, ring_u32 + n_slot * STAGE_BYTES, ring + n_slot * STAGE_BYTES,
                         left - WARPS * kTok, p.qk_scale, lane);
          Policy::update(acc, qs, sc_cur, ring_u32 + c_slot * STAGE_BYTES, ring + c_slot * STAGE_BYTES,
                         left, lane);
          sc_cur = sc_next;
          left -= WARPS * kTok;
          c_slot = n_slot;
          c_phase = n_phase;
        }
        if (!timed_out) {
          __syncwarp();
          issue_next();
          Policy::update(acc, qs, sc_cur, ring_u32 + c_slot * STAGE_BYTES, ring + c_slot * STAGE_BYTES,
                         left, lane);
          if (++c_slot == STAGES) {
            c_slot = 0;
            c_phase ^= 1;
          }
        }
      }
    } else {
      // One tile at a time: scores then update on the same stage, which is refilled (STAGES
      // tiles ahead) as soon as its tile is finished -- except after the segment's last tile:
      // that stage carries the warp's partial through the epilogue and is refilled after it.
      // The body exists once per ring slot, so every shared-memory address in it is a
      // compile-time offset from the warp's ring.
      auto tile = [&](auto slot_c, bool last) {
        constexpr int SL = decltype(slot_c)::value;
        if (!mbar_wait_bounded(bar_u32 + 8 * SL, c_phase)) {
          timed_out = true;
          return;
        }
        __syncwarp();
        typename Policy::Scores sc_cur;
        Policy::scores(sc_cur, qs, ring_u32 + SL * STAGE_BYTES, ring + SL * STAGE_BYTES, left,
                       p.qk_scale, lane);
        Policy::update(acc, qs, sc_cur, ring_u32 + SL * STAGE_BYTES, ring + SL * STAGE_BYTES, left,
                       lane);
        left -= WARPS * kTok;
        if constexpr (SL == STAGES - 1) c_phase ^= 1;
        c_slot = (SL + 1 == STAGES) ? 0 : SL + 1;
        __syncwarp();
        if (!last) issue_at(SL);  // in ring order the next issue always refills the slot just consumed
      };
      for (int i = 0; i < my_tiles && !timed_out; ++i) {
        const bool last = i + 1 == my_tiles;
        if (c_slot == 0) {
          tile(std::integral_constant<int, 0>{}, last);
        } else if (STAGES == 2 || c_slot == 1) {
          tile(std::integral_constant<int, 1>{}, last);
        } else {
          tile(std::integral_constant<int, STAGES - 1>{}, last);
        }
      }
      deferred_issue = my_tiles > 0 && !timed_out;
    }

    // ---- segment epilogue: merge the warps, store the partial ----
    const int vals_slot = (c_slot == 0 ? STAGES : c_slot) - 1;  // the stage consumed last
    float* vals = reinterpret_cast<float*>(ring + vals_slot * STAGE_BYTES);
    SoftmaxState st;
    if (my_tiles > 0) {
      Policy::finalize(acc, vals, st, lane);  // the stage consumed last is free until the next issue
    } else {
      st = SoftmaxState{-INFINITY, -INFINITY, 0.f, 0.f};
    }
    if ((lane >> 2) == 0) {
      const int t = lane & 3;
      s_m[warp][2 * t] = st.m0;
      s_m[warp][2 * t + 1] = st.m1;
      s_l[warp][2 * t] = st.l0;
      s_l[warp][2 * t + 1] = st.l1;
    }
    if (lane == 0) s_slot[warp] = vals_slot;
    __syncthreads();
    // Each thread merges float4 columns; per item the four warps' loads are independent
    // (no data-dependent branch around them), so they overlap instead of serialising.
    {
      constexpr int D4 = D / 4;
      constexpr int ITEMS = kHeadsPerCta * D4;
      constexpr int ROUNDS = (ITEMS + WARPS * 32 - 1) / (WARPS * 32);
      uint32_t voff[WARPS];
#pragma unroll
      for (int w = 0; w < WARPS; ++w) voff[w] = (uint32_t)((w * STAGES + s_slot[w]) * STAGE_BYTES);
#pragma unroll
      for (int it = 0; it < ROUNDS; ++it) {
        const int idx = it * (WARPS * 32) + threadIdx.x;
        if (ITEMS % (WARPS * 32) != 0 && idx >= ITEMS) break;
        const int h = idx / D4, d = (idx - h * D4) * 4;
        const int hg = seg.hc * kHeadsPerCta + h;
        if (hg >= p.group) continue;
        float mw[WARPS], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          mw[w] = s_m[w][h];
          M = fmaxf(M, mw[w]);
        }
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const bool live = mw[w] != -INFINITY;  // a warp without tiles left its stage unwritten
          const float s = live ? ex2(mw[w] - M) : 0.f;
          const float4 v = *reinterpret_cast<const float4*>(smem + voff[w] + (h * D + d) * 4);
          a.x = fmaf(s, live ? v.x : 0.f, a.x);
          a.y = fmaf(s, live ? v.y : 0.f, a.y);
          a.z = fmaf(s, live ? v.z : 0.f, a.z);
          a.w = fmaf(s, live ? v.w : 0.f, a.w);
          L = fmaf(s, s_l[w][h], L);
        }
        const int64_t hq = (int64_t)seg.b * p.HQ + seg.hkv * p.group + hg;
        if (p.partials) {
          const int64_t pi = hq * sc.nslots + seg.slot;
          *reinterpret_cast<float4*>(p.acc + pi * D + d) = a;
          if (d == 0) {
            p.m[pi] = M;
            p.l[pi] = L;
          }
        } else {
          const float inv = (L > 0.f) ? 1.f / L : 0.f;
          *reinterpret_cast<float4*>(p.out + hq * D + d) =
              make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
      }
    }
    if (kMulti && seg.fill_from >= 0) {
      // this CTA finished the unit: mark the unit's unused partial slots empty
      const int nfill = seg.fill_to - seg.fill_from;
      for (int idx = threadIdx.x; idx < kHeadsPerCta * nfill; idx += WARPS * 32) {
        const int h = idx / nfill, j = idx - h * nfill;
        const int hg = seg.hc * kHeadsPerCta + h;
        if (hg < p.group) {
          const int64_t hq = (int64_t)seg.b * p.HQ + seg.hkv * p.group + hg;
          p.m[hq * sc.nslots + seg.fill_from + j] = -INFINITY;
          p.l[hq * sc.nslots + seg.fill_from + j] = 0.f;
        }
      }
    }
    __syncthreads();
    need_proxy_fence = true;
    if (!Policy::PIPELINED && deferred_issue) issue_next();

    if constexpr (!kMulti) {
      break;
    } else {
      g = seg.g_end;
      if (g >= g1 || timed_out) break;
      seg = seg_at(g, g1);
      if (seg.g_end < g1) {  // the query slot just released takes the segment after the next
        const Segment s2 = seg_at(seg.g_end, g1);
        prefetch_q(seg_k & 1, s2.b, s2.hkv, s2.hc);
      }
      ++seg_k;
    }
  }
  if (timed_out && lane == 0) Policy::report_timeout();
}


// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Tensor map over a row-major byte matrix [rows, row_bytes] whose box is
// [box_rows, box_bytes] starting at byte column c0 (given at load time), with the
// shared-memory swizzle that makes 8-row x 16-byte ldmatrix blocks conflict free.
inline int make_row_map(CUtensorMap* tm, const void* base, int64_t rows, int row_bytes,
                        int box_bytes, int box_rows) {
  // A decode loop encodes the same few maps every step: keep the last ones per thread.
  struct Entry {
    const void* base;
    int64_t rows;
    int row_bytes, box_bytes, box_rows;
    CUtensorMap map;
  };
  constexpr int kEntries = 8;
  thread_local Entry cache[kEntries] = {};
  thread_local int next = 0;
  for (int i = 0; i < kEntries; ++i) {
    const Entry& e = cache[i];
    if (e.base == base && e.rows == rows && e.row_bytes == row_bytes && e.box_bytes == box_bytes &&
        e.box_rows == box_rows) {
      *tm = e.map;
      return TKV_OK;
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  TKV_REQUIRE(fn != nullptr, TKV_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  const cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle swz = box_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                 : box_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                   : CU_TENSOR_MAP_SWIZZLE_NONE;
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim,
                        gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TKV_REQUIRE(r == CUDA_SUCCESS, TKV_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
              (int)r);
  Entry& e = cache[next];
  next = (next + 1) % kEntries;
  e.base = base;
  e.rows = rows;
  e.row_bytes = row_bytes;
  e.box_bytes = box_bytes;
  e.box_rows = box_rows;
  e.map = *tm;
  return TKV_OK;
}

// One map over two byte matrices [rows, 128] that lie `gap` bytes apart (the lower one first):
// dims {128, rows, 2}, box {128, box_rows, 2}, 128-byte swizzle.
inline int make_pair_map(CUtensorMap* tm, const void* lower, uint64_t gap, int64_t rows, int box_rows) {
  // A decode loop encodes the same map every step: keep the last ones per thread.
  struct Entry {
    const void* lower;
    uint64_t gap;
    int64_t rows;
    int box_rows;
    CUtensorMap map;
  };
  constexpr int kEntries = 4;
  thread_local Entry cache[kEntries] = {};
  thread_local int next = 0;
  for (int i = 0; i < kEntries; ++i) {
    const Entry& e = cache[i];
    if (e.lower == lower && e.gap == gap && e.rows == rows && e.box_rows == box_rows && e.lower != nullptr) {
      *tm = e.map;
      return TKV_OK;
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  TKV_REQUIRE(fn != nullptr, TKV_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  const cuuint64_t gdim[3] = {128, (cuuint64_t)rows, 2};
  const cuuint64_t gstride[2] = {128, (cuuint64_t)gap};
  const cuuint32_t box[3] = {128, (cuuint32_t)box_rows, 2};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(lower), gdim, gstride, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TKV_REQUIRE(r == CUDA_SUCCESS, TKV_ERR_CUDA, "cuTensorMapEncodeTiled (pair) failed with CUresult %d", (int)r);
  Entry& e = cache[next];
  next = (next + 1) % kEntries;
  e.lower = lower;
  e.gap = gap;
  e.rows = rows;
  e.box_rows = box_rows;
  e.map = *tm;
  return TKV_OK;
}

// MODES: bit m set = schedule mode m (1, 2, 3) is built for this policy.
template <class Policy, int MODES = 0xE>
struct SplitLaunch {
  static constexpr bool kHas1 = (MODES & 2) != 0, kHas2 = (MODES & 4) != 0, kHas3 = (MODES & 8) != 0;
  static_assert(kHas1 || kHas2 || kHas3, "no schedule mode selected");
  static int smem_bytes() {
    return Policy::WARPS * Policy::STAGES * Policy::STAGE_BYTES + Policy::WARPS * Policy::STAGES * 8 +
           16 + 2 * kHeadsPerCta * Policy::D * 4 +  // query barriers and the two query slots
           Policy::QFRAG_BYTES +                    // query fragments shared by the warps
           1024;                                    // slack for the 1024-byte alignment of the ring
  }
  static constexpr int kPrefixBytes = (kMaxRaggedB + 1) * 4 + 32;  // ragged batches: tile prefix
  template <int MODE>
  static const void* fn_mode() { return reinterpret_cast<const void*>(&splitk_kernel<Policy, MODE>); }
  // same launch bounds and shared memory in all modes: any built one answers for the family
  static const void* fn() {
    if constexpr (kHas1) return fn_mode<1>();
    else if constexpr (kHas2) return fn_mode<2>();
    else return fn_mode<3>();
  }
  static int prepare() {
    static bool done[64] = {};
    int dev = 0;
    TKV_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && done[dev]) return TKV_OK;
    if constexpr (kHas1)
      TKV_CUDA(cudaFuncSetAttribute(fn_mode<1>(), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes()));
    if constexpr (kHas2)
      TKV_CUDA(cudaFuncSetAttribute(fn_mode<2>(), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes()));
    if constexpr (kHas3)
      TKV_CUDA(cudaFuncSetAttribute(fn_mode<3>(), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    smem_bytes() + kPrefixBytes));
    if (dev < 64) done[dev] = true;
    return TKV_OK;
  }
  // CTAs resident at once on the current device (one wave of the persistent grid).
  static int wave(int* out) {
    static int cached[64] = {};
    int dev = 0;
    TKV_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && cached[dev] > 0) {
      *out = cached[dev];
      return TKV_OK;
    }
    int rc = prepare();
    if (rc != TKV_OK) return rc;
    int n = 0, sms = 0;
    TKV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn(), Policy::WARPS * 32,
                                                           smem_bytes()));
    TKV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    TKV_REQUIRE(n > 0 && sms > 0, TKV_ERR_CUDA, "split kernel does not fit on this device");
    *out = n * sms;
    if (dev < 64) cached[dev] = *out;
    return TKV_OK;
  }
  static int plan(SplitSched* sc, int B, int HKV, int hchunks, int S, int num_splits,
                  int split_size, bool ragged) {
    int w = 0;
    int rc = wave(&w);
    if (rc != TKV_OK) return rc;
    *sc = make_sched(B, HKV, hchunks, S, num_splits, split_size, ragged, w, Policy::TOK,
                     Policy::WARPS, kHas2);
    return TKV_OK;
  }
  static int launch(const typename Policy::Maps& maps, const DecodeParams& p, const SplitSched& sc,
                    cudaStream_t stream) {
    int rc = prepare();
    if (rc != TKV_OK) return rc;
    // The kernel is launched as a programmatic dependent: its prologue overlaps the tail of the
    // previous kernel of the stream and it waits for that kernel's completion before its first
    // global access.  For unit-aligned plans (small batches, CTAs of a few microseconds) the
    // preceding combine kernel lets its dependents go at its start.  The balanced global plan
    // has CTAs that run for tens of microseconds and must all be resident together: a CTA that
    // found its place taken by a still-resident combine CTA started 10-30 us late (measured),
    // which the static tile ranges cannot absorb -- so the combine kernel used behind that
    // plan (the warp-per-row one) lets its dependents go only when its own work is done, and
    // what overlaps is the launch itself (batch 8: 17.6 -> 16.8 us per step, batch 64: -0.3 %).
    const dim3 grid(sc.grid), block(Policy::WARPS * 32);
    if (sc.persistent == 1) {
      if constexpr (kHas1) {
        // (dependent only where the combine behind the previous step is the one that waits)
        if (sc.nslots > 1 && sc.nslots <= kSmallCombineMaxSlots && (int64_t)p.B * p.HQ >= kSmallCombineMinRows) {
          TKV_CUDA(launch_pdl(splitk_kernel<Policy, 1>, grid, block, (size_t)smem_bytes(), stream, maps, p, sc));
        } else {
          splitk_kernel<Policy, 1><<<grid, block, smem_bytes(), stream>>>(maps, p, sc);
          TKV_CUDA(cudaGetLastError());
        }
        return TKV_OK;
      }
    } else if (sc.persistent == 3) {
      if constexpr (kHas3) {
        splitk_kernel<Policy, 3><<<grid, block, smem_bytes() + kPrefixBytes, stream>>>(maps, p, sc);
        TKV_CUDA(cudaGetLastError());
        return TKV_OK;
      }
    } else if constexpr (kHas2) {
      if (sc.persistent == 2) {
        TKV_CUDA(launch_pdl(splitk_kernel<Policy, 2>, grid, block, (size_t)smem_bytes(), stream, maps, p, sc));
      } else {
        splitk_kernel<Policy, 2><<<grid, block, smem_bytes(), stream>>>(maps, p, sc);
        TKV_CUDA(cudaGetLastError());
      }
      return TKV_OK;
    }
    set_error("split kernel: schedule mode %d is not built for this kernel family", sc.persistent);
    return TKV_ERR_INVALID;
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
      TKV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn(), Policy::WARPS * 32,
                                                             smem_bytes()));
      *ctas = n;
    }
    return TKV_OK;
  }
};

// Argument checks and DecodeParams fields shared by the two decode entry points.
inline int fill_common(DecodeParams& p, const char* who, const void* q, int q_dtype, float* acc,
                       float* m, float* l, float* out, int B, int HQ, int HKV, int S,
                       float sm_scale, int num_splits, int split_size, int nslots,
                       const int32_t* seq_lens, int flags) {
  TKV_REQUIRE(B > 0 && HQ > 0 && HKV > 0 && S > 0, TKV_ERR_INVALID,
              "%s: B, HQ, HKV, S must be positive (got %d, %d, %d, %d)", who, B, HQ, HKV, S);
  TKV_REQUIRE((int64_t)B * HKV * S < (1LL << 31), TKV_ERR_INVALID,
              "%s: B*HKV*S = %lld cached tokens exceed 2^31", who, (long long)B * HKV * S);
  TKV_REQUIRE(HQ % HKV == 0, TKV_ERR_INVALID, "HQ=%d must be a multiple of HKV=%d", HQ, HKV);
  TKV_REQUIRE(q_dtype >= 0 && q_dtype <= 2, TKV_ERR_INVALID, "%s: bad q dtype %d", who, q_dtype);
  TKV_REQUIRE(num_splits >= 1 && split_size >= 16 && split_size % 16 == 0, TKV_ERR_INVALID,
              "%s: split_size=%d must be a positive multiple of 16, num_splits=%d >= 1", who,
              split_size, num_splits);
  TKV_REQUIRE((int64_t)num_splits * split_size >= S &&
                  (int64_t)(num_splits - 1) * split_size < S,
              TKV_ERR_INVALID, "%s: %d splits of %d tokens must cover S=%d with no empty split", who,
              num_splits, split_size, S);
  const bool partials = nslots > 1 || (flags & TKV_FLAG_PARTIALS_ONLY);
  TKV_REQUIRE(!partials || (acc && m && l), TKV_ERR_INVALID,
              "%s: partial buffers (acc, m, l) required", who);
  TKV_REQUIRE(partials || out, TKV_ERR_INVALID, "%s: out required", who);
  TKV_REQUIRE(aligned16(q), TKV_ERR_ALIGN, "%s: q must be 16-byte aligned", who);
  TKV_REQUIRE(aligned16(acc) && aligned16(out), TKV_ERR_ALIGN,
              "%s: acc and out must be 16-byte aligned", who);
  p.q = q;
  p.q_dtype = q_dtype;
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
  return TKV_OK;
}

}  // namespace tkv
