// Group-wise quantiser and split-P packing kernels (sm_100a).
//
// Replaces the eager PyTorch chain of the reference's quantize.py with one launch
// each: pack_codes (:149-169), unpack_codes (:172-183), quantize_groupwise (:186-236),
// dequantize_groupwise (:239-246).  Integer and rounding behaviour is bit-exact:
// every float operation below is a single IEEE round-to-nearest operation written
// with an explicit intrinsic so that neither FMA contraction nor a fast-math flag
// can change it.
#include <type_traits>

#include "tkv_common.cuh"

namespace tkv {

// ---------------------------------------------------------------- quantize + pack
// Each thread owns E consecutive elements of a row (E = 16 for f16/bf16 rows: two 16-byte loads;
// E = 8 otherwise), in kRowsPerThread rows.  A quantisation group spans GS/E adjacent lanes; min
// and max are butterfly-reduced inside it as the pair (min, -max) with a NaN-propagating
// minimum -- for 16-bit inputs as ONE packed half2 per shuffle.  The codes of a thread are E/4
// 32-bit words (one code per byte); split-P packing ORs the words of the P lanes that hold
// dims j, j+DP, ... shifted by their bit-slice position.  Every size is a power of two, so all
// index arithmetic is shifts.
//
// Codes.  The reference computes round((x - zero) / scale) with an IEEE division.  Here the
// quotient is a * (1/scale): within 1e-5 of the IEEE quotient wherever the clamp does not
// decide the code (|q| <= 17), so it rounds to the same integer unless it lies within 1e-4 of
// a half-integer -- those elements (about one in 1500 for f16 data, whose quotients hit exact
// ties) are redone with the IEEE division.  Bit-exact, at a fifth of the instructions.
// The scale's division by 2^nbits - 1 is q0 = d*R, q1 = fma(fma(-q0, QMAX, d), R, q0) with R the
// rounded reciprocal: the correctly rounded quotient for every finite d (checked against the
// IEEE division over 160 M values of d, all fp16 values among them).
constexpr int kRowsPerThread = 2;

__device__ __forceinline__ float min_nan(float a, float b) {
  float d;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ float rcp_approx(float a) {
  float d;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(d) : "f"(a));
  return d;
}

// A thread's E elements as f32 plus their (min, -max); NaN propagates to both (torch's
// amin/amax do; fminf/fmaxf would drop it).  For 16-bit types the pair stays a packed half2.
template <typename T>
struct Pair16;
template <>
struct Pair16<__half> { using type = __half2; };
template <>
struct Pair16<__nv_bfloat16> { using type = __nv_bfloat162; };

template <typename H2>
__device__ __forceinline__ float2 widen2(H2 h);
template <>
__device__ __forceinline__ float2 widen2<__half2>(__half2 h) { return __half22float2(h); }
template <>
__device__ __forceinline__ float2 widen2<__nv_bfloat162>(__nv_bfloat162 h) { return __bfloat1622float2(h); }

// (min over both halves of a, -max over both halves of b) as one packed pair
template <typename H2>
__device__ __forceinline__ H2 fold_minmax(H2 a, H2 b) {
  b = __hneg2(b);
  const uint32_t au = *reinterpret_cast<const uint32_t*>(&a), bu = *reinterpret_cast<const uint32_t*>(&b);
  const uint32_t lo = __byte_perm(au, bu, 0x5410), hi = __byte_perm(au, bu, 0x7632);  // (a.x, b.x), (a.y, b.y)
  return __hmin2_nan(*reinterpret_cast<const H2*>(&lo), *reinterpret_cast<const H2*>(&hi));
}

// (x.lo - z, x.hi - z) in f32 from a packed pair of 16-bit values: the mixed-precision subtract of
// sm_100 widens the 16-bit operand itself, so no conversion instruction is spent per element.
template <typename H2>
__device__ __forceinline__ float2 sub_widen(H2 x, float z);
template <>
__device__ __forceinline__ float2 sub_widen<__half2>(__half2 x, float z) {
  float2 r;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tsub.rn.f32.f16 %0, l, %3;\n\tsub.rn.f32.f16 %1, h, %3;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "r"(*reinterpret_cast<const uint32_t*>(&x)), "f"(z));
  return r;
}
template <>
__device__ __forceinline__ float2 sub_widen<__nv_bfloat162>(__nv_bfloat162 x, float z) {
  float2 r;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tsub.rn.f32.bf16 %0, l, %3;\n\tsub.rn.f32.bf16 %1, h, %3;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "r"(*reinterpret_cast<const uint32_t*>(&x)), "f"(z));
  return r;
}

// Where the rows go when new tokens are appended to a preallocated cache (cap == 0: in place).
struct AppendMap {
  const int32_t* pos;  // per-sequence first free slot, or null for pos0 everywhere
  int pos0;
  int t_new;           // new tokens per (sequence, head)
  int hkv;             // heads per sequence
  int64_t cap;         // token rows per (sequence, head) in the cache
};

// `tpr_shift` = log2(D/E) (threads per row), `lpg_shift` = log2(GS/E) (lanes per group).  Block
// b handles rows [b*RPB, (b+1)*RPB) with RPB = kRowsPerThread * 256 / tpr, thread t the column
// block t % tpr of rows b*RPB + t/tpr + i*(256/tpr).
template <typename T, int NBITS, int E>
__global__ void __launch_bounds__(256)
    quantize_pack_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed,
                         __half* __restrict__ scale, __half* __restrict__ zero, int64_t rows,
                         int tpr_shift, int lpg_shift, const AppendMap am) {
  constexpr int LOG2P = NBITS == 4 ? 1 : 2;  // P = 8 / NBITS codes per packed byte
  constexpr float QMAX = float((1 << NBITS) - 1);
  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: x + kMagic holds rint(x) in its low mantissa bits
  constexpr bool k16 = !std::is_same<T, float>::value;
  static_assert(E == 8 || (E == 16 && k16), "16 elements per thread are two 16-byte loads of a 16-bit type");
  const int tpr = 1 << tpr_shift;
  const int c = threadIdx.x & (tpr - 1);            // E-element column block
  const int rstep = 256 >> tpr_shift;               // rows of one pass of the block
  const int64_t row0 = (int64_t)blockIdx.x * (kRowsPerThread * rstep) + (threadIdx.x >> tpr_shift);
  const int lanes_per_group = 1 << lpg_shift;
  const int tps_shift = tpr_shift - LOG2P;          // lanes per bit slice
  const int p = c >> tps_shift;
  const int D = E << tpr_shift;
#pragma unroll
  for (int it = 0; it < kRowsPerThread; ++it) {
    const int64_t row = row0 + it * rstep;
    const bool live = row < rows;
    // Lanes past the end mirror the last row so the shuffles below stay full-warp.
    const int64_t r = live ? row : rows - 1;
    const T* src = x + r * D + E * c;
    float a[E], mn, nmx;  // a: the elements (f32 rows) and then x - zero
    [[maybe_unused]] uint32_t raw[k16 ? E / 2 : 1];  // 16-bit rows: the elements as loaded
    if constexpr (k16) {
      using H2 = typename Pair16<T>::type;
      H2 h[E / 2];
#pragma unroll
      for (int i = 0; i < E / 8; ++i)
        *reinterpret_cast<uint4*>(&h[4 * i]) = __ldg(reinterpret_cast<const uint4*>(src) + i);
      H2 lo = h[0], hi = h[0];
#pragma unroll
      for (int i = 1; i < E / 2; ++i) {
        lo = __hmin2_nan(lo, h[i]);
        hi = __hmax2_nan(hi, h[i]);
      }
      H2 pm = fold_minmax<H2>(lo, hi);
      for (int off = 1; off < lanes_per_group; off <<= 1) {
        const uint32_t o = __shfl_xor_sync(kFullMask, *reinterpret_cast<const uint32_t*>(&pm), off);
        pm = __hmin2_nan(pm, *reinterpret_cast<const H2*>(&o));
      }
      const float2 f = widen2<H2>(pm);
      mn = f.x;
      nmx = f.y;
#pragma unroll
      for (int i = 0; i < E / 2; ++i) raw[i] = *reinterpret_cast<const uint32_t*>(&h[i]);
    } else {
      const float4 lo4 = __ldg(reinterpret_cast<const float4*>(src));
      const float4 hi4 = __ldg(reinterpret_cast<const float4*>(src) + 1);
      a[0] = lo4.x; a[1] = lo4.y; a[2] = lo4.z; a[3] = lo4.w;
      a[4] = hi4.x; a[5] = hi4.y; a[6] = hi4.z; a[7] = hi4.w;
      mn = a[0];
      nmx = -a[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) {
        mn = min_nan(mn, a[i]);
        nmx = min_nan(nmx, -a[i]);
      }
      for (int off = 1; off < lanes_per_group; off <<= 1) {
        mn = min_nan(mn, __shfl_xor_sync(kFullMask, mn, off));
        nmx = min_nan(nmx, __shfl_xor_sync(kFullMask, nmx, off));
      }
    }
    // A group that holds a NaN gets zero = NaN, scale = 1 and all codes 0, as the reference produces.
    const float range = __fsub_rn(-nmx, mn);
    const float q0 = __fmul_rn(range, 1.f / QMAX);
    const float q1 = __fmaf_rn(__fmaf_rn(-q0, QMAX, range), 1.f / QMAX, q0);
    float sc = range == INFINITY ? range : q1;  // = __fdiv_rn(range, QMAX)
    sc = (sc > 0.f) ? sc : 1.f;
    const __half sc16 = __float2half_rn(sc);
    const __half ze16 = __float2half_rn(mn);
    const float scf = __half2float(sc16), zef = __half2float(ze16);
    const float rs = __fmul_rn(rcp_approx(scf), 1.f / QMAX);  // a * rs = quotient / QMAX, saturated to [0, 1]

    if constexpr (k16) {
      using H2 = typename Pair16<T>::type;
#pragma unroll
      for (int i = 0; i < E / 2; ++i) {
        const float2 d = sub_widen<H2>(*reinterpret_cast<const H2*>(&raw[i]), zef);
        a[2 * i] = d.x;
        a[2 * i + 1] = d.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) a[i] = __fsub_rn(a[i], zef);
    }
    float m[E];
    uint32_t near_tie = 0;  // bit i: element i lies next to a tie
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float u = __saturatef(__fmul_rn(a[i], rs));                  // NaN -> 0, as the clamp gives
      m[i] = __fmaf_rn(u, QMAX, kMagic);
      const float d = __fmaf_rn(u, QMAX, -__fsub_rn(m[i], kMagic));      // distance to the integer taken
      if (fabsf(d) > 0.4999f) near_tie |= 1u << i;
    }
    uint32_t w[E / 4];  // codes, one per byte
#pragma unroll
    for (int i = 0; i < E / 4; ++i) {
      const uint32_t lo2 = __byte_perm(__float_as_uint(m[4 * i]), __float_as_uint(m[4 * i + 1]), 0x0040);
      const uint32_t hi2 = __byte_perm(__float_as_uint(m[4 * i + 2]), __float_as_uint(m[4 * i + 3]), 0x0040);
      w[i] = __byte_perm(lo2, hi2, 0x5410);
    }
    // About one thread in a hundred has such an element (a third of the warps): those codes are
    // redone with the IEEE division from the element as stored and put into their byte.
    while (near_tie) {
      const int i = __ffs(near_tie) - 1;
      near_tie &= near_tie - 1;
      float xi;
      if constexpr (std::is_same<T, float>::value) {
        xi = src[i];
      } else if constexpr (std::is_same<T, __half>::value) {
        xi = __half2float(src[i]);
      } else {
        xi = __bfloat162float(src[i]);
      }
      float t = rintf(__fdiv_rn(__fsub_rn(xi, zef), scf));
      t = fminf(fmaxf(t, 0.f), QMAX);
      const uint32_t sh = (i & 3) * 8, code = (uint32_t)(int)t << sh, byte = 0xffu << sh;
#pragma unroll
      for (int k = 0; k < E / 4; ++k) {  // masks, not an indexed store: w stays in registers
        const uint32_t sel = (k == (i >> 2)) ? byte : 0u;
        w[k] = (w[k] & ~sel) | (code & sel);
      }
    }
#pragma unroll
    for (int i = 0; i < E / 4; ++i) w[i] <<= (NBITS * p);
    // split-P: lane c = p*TPS + c' contributes bit slice p of bytes [E*c', E*c' + E)
    for (int off = 1 << tps_shift; off < tpr; off <<= 1) {
#pragma unroll
      for (int i = 0; i < E / 4; ++i) w[i] |= __shfl_xor_sync(kFullMask, w[i], off);
    }
    // Output row: the input row itself, or (append) slot pos[b] + t of sequence (b, head)
    // in a cache of `cap` token rows per sequence; tokens that fall outside are dropped.
    int64_t orow = row;
    bool keep = live;
    if (am.cap > 0 && live) {
      int64_t bh;
      int t;
      if (rows < (1LL << 31)) {  // 32-bit divisions: a 64-bit one is tens of instructions per thread
        const uint32_t q = (uint32_t)row / (uint32_t)am.t_new;
        bh = q;
        t = (int)((uint32_t)row - q * (uint32_t)am.t_new);
      } else {
        bh = row / am.t_new;
        t = (int)(row - bh * am.t_new);
      }
      const int64_t at = (am.pos ? (int64_t)am.pos[(uint32_t)bh / (uint32_t)am.hkv] : (int64_t)am.pos0) + t;
      keep = at >= 0 && at < am.cap;
      orow = bh * am.cap + at;
    }
    if (keep) {
      if (p == 0) {
        uint8_t* dst = packed + orow * (D >> LOG2P) + E * c;
        if constexpr (E == 16) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
          *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
        }
      }
      if ((c & (lanes_per_group - 1)) == 0) {
        const int64_t gi = (orow << (tpr_shift - lpg_shift)) + (c >> lpg_shift);
        scale[gi] = sc16;
        zero[gi] = ze16;
      }
    }
  }
}

// ---------------------------------------------------------------- per-channel keys
// Keys quantised per channel: a group is kChanTok consecutive tokens of ONE head dimension
// (the reference describes the format as future work, docs/future_work.md:229-293, and has
// no implementation of it).  Same per-element arithmetic as quantize_pack_kernel on the other
// axis; the codes keep the split-P byte layout along the head dimension, scale and zero are
// one row of D values per block of kChanTok tokens.
// A CTA of 256 threads takes 512/D consecutive token blocks; a thread owns two adjacent head
// dimensions of one block and walks its 32 tokens (4-byte loads of a 16-bit row, contiguous
// across the warp), keeps min and max per dimension as packed pairs, derives the two scales and
// zeros, leaves its codes in shared memory, and the CTA then packs whole rows, 16 bytes per
// thread and store.
constexpr int kChanTok = 32;

// One dimension's scale, zero and reciprocal from its (min, max).
struct ChanScale {
  __half sc16, ze16;
  float scf, zef, rs;
};
template <int NBITS>
__device__ __forceinline__ ChanScale chan_scale(float mn, float mx) {
  constexpr float QMAX = float((1 << NBITS) - 1);
  ChanScale r;
  float sc = __fdiv_rn(__fsub_rn(mx, mn), QMAX);
  sc = (sc > 0.f) ? sc : 1.f;
  r.sc16 = __float2half_rn(sc);
  r.ze16 = __float2half_rn(mn);
  r.scf = __half2float(r.sc16);
  r.zef = __half2float(r.ze16);
  r.rs = __fmul_rn(rcp_approx(r.scf), 1.f / QMAX);
  return r;
}

// The two elements of one token as f32 (the loads of the second pass hit L1/L2).
template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 load2<__half>(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

template <typename T, int NBITS>
__global__ void __launch_bounds__(256)
    quantize_keys_channel_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed,
                                 __half* __restrict__ scale, __half* __restrict__ zero,
                                 int64_t S, int64_t S_q, int D, int64_t n_blocks) {
  constexpr int P = 8 / NBITS;
  constexpr float QMAX = float((1 << NBITS) - 1);
  constexpr float kMagic = 12582912.f;
  constexpr bool k16 = !std::is_same<T, float>::value;
  __shared__ __align__(16) uint8_t codes[512 * kChanTok];  // [local block][token][dim]
  const int tpb = D >> 1;                                   // threads per token block
  const int nb = 256 / tpb;                                 // token blocks per CTA
  const int lb = threadIdx.x / tpb, dp = threadIdx.x - lb * tpb;
  const int64_t blocks_per_seq = S_q / kChanTok;
  const int64_t gb = (int64_t)blockIdx.x * nb + lb;
  if (gb < n_blocks) {
    const int64_t bh = gb / blocks_per_seq, tb = gb - bh * blocks_per_seq;
    const T* src = x + (bh * S + tb * kChanTok) * D + 2 * dp;
    float mn0, mn1, mx0, mx1;
    [[maybe_unused]] uint32_t raw[k16 ? kChanTok : 1];
    if constexpr (k16) {
      using H2 = typename Pair16<T>::type;
      H2 lo, hi;
#pragma unroll
      for (int t = 0; t < kChanTok; ++t) {
        raw[t] = __ldg(reinterpret_cast<const uint32_t*>(src + (int64_t)t * D));
        const H2 h = *reinterpret_cast<const H2*>(&raw[t]);
        lo = t == 0 ? h : __hmin2_nan(lo, h);  // NaN propagates, as in the per-token quantiser
        hi = t == 0 ? h : __hmax2_nan(hi, h);
      }
      const float2 l = widen2<H2>(lo), u = widen2<H2>(hi);
      mn0 = l.x; mn1 = l.y; mx0 = u.x; mx1 = u.y;
    } else {
      float n0, n1;  // -max
#pragma unroll
      for (int t = 0; t < kChanTok; ++t) {
        const float2 v = __ldg(reinterpret_cast<const float2*>(src + (int64_t)t * D));
        mn0 = t == 0 ? v.x : min_nan(mn0, v.x);
        mn1 = t == 0 ? v.y : min_nan(mn1, v.y);
        n0 = t == 0 ? -v.x : min_nan(n0, -v.x);
        n1 = t == 0 ? -v.y : min_nan(n1, -v.y);
      }
      mx0 = -n0;
      mx1 = -n1;
    }
    const ChanScale c0 = chan_scale<NBITS>(mn0, mx0), c1 = chan_scale<NBITS>(mn1, mx1);
    const int64_t mrow = gb * D + 2 * dp;
    *reinterpret_cast<__half2*>(scale + mrow) = __halves2half2(c0.sc16, c1.sc16);
    *reinterpret_cast<__half2*>(zero + mrow) = __halves2half2(c0.ze16, c1.ze16);
    // codes by the reciprocal, those next to a tie redone with the IEEE division (see
    // quantize_pack_kernel)
    uint8_t* crow = codes + (lb * kChanTok) * D + 2 * dp;
    uint32_t near_tie = 0;  // bit t: token t holds a code next to a tie
#pragma unroll
    for (int t = 0; t < kChanTok; ++t) {
      float a0, a1;
      if constexpr (k16) {
        using H2 = typename Pair16<T>::type;
        const float2 v = widen2<H2>(*reinterpret_cast<const H2*>(&raw[t]));
        a0 = __fsub_rn(v.x, c0.zef);
        a1 = __fsub_rn(v.y, c1.zef);
      } else {
        const float2 v = __ldg(reinterpret_cast<const float2*>(src + (int64_t)t * D));
        a0 = __fsub_rn(v.x, c0.zef);
        a1 = __fsub_rn(v.y, c1.zef);
      }
      const float u0 = __saturatef(__fmul_rn(a0, c0.rs)), u1 = __saturatef(__fmul_rn(a1, c1.rs));
      const float m0 = __fmaf_rn(u0, QMAX, kMagic), m1 = __fmaf_rn(u1, QMAX, kMagic);
      const float d0 = __fmaf_rn(u0, QMAX, -__fsub_rn(m0, kMagic));
      const float d1 = __fmaf_rn(u1, QMAX, -__fsub_rn(m1, kMagic));
      if (fabsf(d0) > 0.4999f || fabsf(d1) > 0.4999f) near_tie |= 1u << t;
      *reinterpret_cast<uint16_t*>(crow + t * D) =
          (uint16_t)__byte_perm(__float_as_uint(m0), __float_as_uint(m1), 0x0040);
    }
    // about one thread in twenty has such a token, so most warps come here -- for one token or two
    while (near_tie) {
      const int t = __ffs(near_tie) - 1;
      near_tie &= near_tie - 1;
      {
        const float2 v = load2<T>(src + (int64_t)t * D);
        float q0 = rintf(__fdiv_rn(__fsub_rn(v.x, c0.zef), c0.scf));
        float q1 = rintf(__fdiv_rn(__fsub_rn(v.y, c1.zef), c1.scf));
        q0 = fminf(fmaxf(q0, 0.f), QMAX);
        q1 = fminf(fmaxf(q1, 0.f), QMAX);
        *reinterpret_cast<uint16_t*>(crow + t * D) = (uint16_t)((int)q0 | ((int)q1 << 8));
      }
    }
  }
  __syncthreads();
  // pack: byte j of a token = OR_p code[j + p*DP] << (p*NBITS); a thread makes 16 bytes at a time
  const int DP = D / P;
  const int chunks_per_row = DP >> 4;  // DP >= 16 (checked by the caller)
  const int n_chunks = nb * kChanTok * chunks_per_row;
  for (int i = threadIdx.x; i < n_chunks; i += 256) {
    const int rowl = i / chunks_per_row, j = (i - rowl * chunks_per_row) << 4;  // row = local block * 32 + token
    const int64_t g = (int64_t)blockIdx.x * nb + rowl / kChanTok;
    if (g >= n_blocks) break;  // local blocks are in order: the rest is past the end too
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const uint4 v = *reinterpret_cast<const uint4*>(codes + rowl * D + p * DP + j);
      w.x |= v.x << (p * NBITS);
      w.y |= v.y << (p * NBITS);
      w.z |= v.z << (p * NBITS);
      w.w |= v.w << (p * NBITS);
    }
    // token blocks of one sequence are contiguous in the quantised part: global row = g*32 + token
    *reinterpret_cast<uint4*>(packed + (g * kChanTok + (rowl % kChanTok)) * DP + j) = w;
  }
}

// ---------------------------------------------------------------- plain pack / unpack
template <int NBITS>
__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed,
                                  int64_t n_out, int D) {
  constexpr int P = 8 / NBITS;
  const int DP = D / P;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const int64_t row = i / DP;
  const int j = (int)(i % DP);
  uint32_t b = 0;
#pragma unroll
  for (int p = 0; p < P; ++p) b |= (uint32_t)codes[row * D + j + p * DP] << (p * NBITS);
  packed[i] = (uint8_t)b;  // wraps modulo 256 like the reference's uint8 shift
}

template <int NBITS>
__global__ void unpack_codes_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes,
                                    int64_t n_out, int D) {
  constexpr int P = 8 / NBITS;
  const int DP = D / P;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const int64_t row = i / D;
  const int d = (int)(i % D);
  codes[i] = (packed[row * DP + d % DP] >> ((d / DP) * NBITS)) & ((1 << NBITS) - 1);
}

// ---------------------------------------------------------------- dequantise
template <typename T>
__device__ __forceinline__ T from_float(float f);
template <>
__device__ __forceinline__ float from_float<float>(float f) { return f; }
template <>
__device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) {
  return __float2bfloat16_rn(f);
}

template <typename T, int NBITS>
__global__ void dequantize_kernel(const uint8_t* __restrict__ packed,
                                  const __half* __restrict__ scale,
                                  const __half* __restrict__ zero, T* __restrict__ out,
                                  int64_t n_out, int D, int gs) {
  constexpr int P = 8 / NBITS;
  const int DP = D / P;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const int64_t row = i / D;
  const int d = (int)(i % D);
  const int code = (packed[row * DP + d % DP] >> ((d / DP) * NBITS)) & ((1 << NBITS) - 1);
  const int64_t gi = row * (D / gs) + d / gs;
  // code*scale is exact in f32 (<= 4 + 11 significant bits), so this is the
  // reference's multiply-then-add with one rounding.
  const float f = __fadd_rn(__fmul_rn((float)code, __half2float(scale[gi])), __half2float(zero[gi]));
  out[i] = from_float<T>(f);
}

// ---------------------------------------------------------------- 8 bytes per thread
// The three kernels above as 8-byte-per-thread forms for rows whose packed width is a multiple
// of 8 bytes (and, for dequantise, groups that are multiples of 8 dims): a thread owns packed
// bytes [8c, 8c+8) of a row, i.e. P runs of 8 consecutive dims [p*DP + 8c, p*DP + 8c + 8).
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_half2(f[0], f[1]);
  v.y = pack_half2(f[2], f[3]);
  v.z = pack_half2(f[4], f[5]);
  v.w = pack_half2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
}

// Items (8 packed bytes each) are dealt to a block kItemsPerThread * 256 at a time, thread t taking
// items t, t + 256, ...: every load of a warp is contiguous and a thread has several in flight.
constexpr int kItemsPerThread = 4;

// item -> (row, column block) with a 32-bit division where the tensor allows it (a 64-bit one is
// tens of instructions)
__device__ __forceinline__ void item_row_col(int64_t it, int tpr, bool small, int64_t& row, int& c) {
  if (small) {
    const uint32_t q = (uint32_t)it / (uint32_t)tpr;
    row = q;
    c = (int)((uint32_t)it - q * (uint32_t)tpr);
  } else {
    row = it / tpr;
    c = (int)(it - row * tpr);
  }
}

template <typename T, int NBITS>
__global__ void __launch_bounds__(256)
    dequantize8_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scale,
                       const __half* __restrict__ zero, T* __restrict__ out, int64_t n_items,
                       int D, int gs) {
  constexpr int P = 8 / NBITS;
  constexpr uint32_t MASK = 0x01010101u * ((1u << NBITS) - 1);
  const int DP = D / P, tpr = DP >> 3, ng = D / gs;
  const bool gs_pow2 = (gs & (gs - 1)) == 0;
  const int gs_shift = __ffs(gs) - 1;
  const int64_t base = (int64_t)blockIdx.x * (kItemsPerThread * 256) + threadIdx.x;
  uint2 w[kItemsPerThread];
  int64_t row[kItemsPerThread];
  int c[kItemsPerThread];
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    const int64_t item = base + k * 256;
    const int64_t it = item < n_items ? item : n_items - 1;
    item_row_col(it, tpr, n_items < (1LL << 31), row[k], c[k]);
    w[k] = __ldg(reinterpret_cast<const uint2*>(packed + row[k] * DP + 8 * c[k]));
  }
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    if (base + k * 256 >= n_items) break;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int d0 = p * DP + 8 * c[k];
      const int64_t gi = row[k] * ng + (gs_pow2 ? d0 >> gs_shift : d0 / gs);
      const float sc = __half2float(scale[gi]), ze = __half2float(zero[gi]);
      const uint32_t lo = (w[k].x >> (p * NBITS)) & MASK, hi = (w[k].y >> (p * NBITS)) & MASK;
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // code*scale is exact in f32 (<= 4 + 11 significant bits), so the fused form is the
        // reference's multiply-then-add with its one rounding
        f[i] = __fmaf_rn((float)((lo >> (8 * i)) & 0xffu), sc, ze);
        f[4 + i] = __fmaf_rn((float)((hi >> (8 * i)) & 0xffu), sc, ze);
      }
      store8<T>(out + row[k] * D + d0, f);
    }
  }
}

template <int NBITS>
__global__ void __launch_bounds__(256)
    pack_codes8_kernel(const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed,
                       int64_t n_items, int D) {
  constexpr int P = 8 / NBITS;
  const int DP = D / P, tpr = DP >> 3;
  const int64_t base = (int64_t)blockIdx.x * (kItemsPerThread * 256) + threadIdx.x;
  uint2 v[kItemsPerThread][P];
  int64_t off[kItemsPerThread];
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    const int64_t item = base + k * 256;
    const int64_t it = item < n_items ? item : n_items - 1;
    int64_t row;
    int c;
    item_row_col(it, tpr, n_items < (1LL << 31), row, c);
    off[k] = row * DP + 8 * c;
#pragma unroll
    for (int p = 0; p < P; ++p)
      v[k][p] = __ldg(reinterpret_cast<const uint2*>(codes + row * D + p * DP + 8 * c));
  }
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    if (base + k * 256 >= n_items) break;
    uint2 w = make_uint2(0u, 0u);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      // a byte's bits shifted past bit 7 are dropped, like the reference's uint8 shift: clear what
      // the 32-bit shift carried into the low bits of the next byte
      const uint32_t keep = ~(0x01010101u * ((1u << (p * NBITS)) - 1));
      w.x |= (v[k][p].x << (p * NBITS)) & keep;
      w.y |= (v[k][p].y << (p * NBITS)) & keep;
    }
    *reinterpret_cast<uint2*>(packed + off[k]) = w;
  }
}

template <int NBITS>
__global__ void __launch_bounds__(256)
    unpack_codes8_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes,
                         int64_t n_items, int D) {
  constexpr int P = 8 / NBITS;
  constexpr uint32_t MASK = 0x01010101u * ((1u << NBITS) - 1);
  const int DP = D / P, tpr = DP >> 3;
  const int64_t base = (int64_t)blockIdx.x * (kItemsPerThread * 256) + threadIdx.x;
  uint2 w[kItemsPerThread];
  int64_t off[kItemsPerThread];
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    const int64_t item = base + k * 256;
    const int64_t it = item < n_items ? item : n_items - 1;
    int64_t row;
    int c;
    item_row_col(it, tpr, n_items < (1LL << 31), row, c);
    off[k] = row * D + 8 * c;
    w[k] = __ldg(reinterpret_cast<const uint2*>(packed + row * DP + 8 * c));
  }
#pragma unroll
  for (int k = 0; k < kItemsPerThread; ++k) {
    if (base + k * 256 >= n_items) break;
#pragma unroll
    for (int p = 0; p < P; ++p)
      *reinterpret_cast<uint2*>(codes + off[k] + p * DP) =
          make_uint2((w[k].x >> (p * NBITS)) & MASK, (w[k].y >> (p * NBITS)) & MASK);
  }
}

inline bool pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

}  // namespace tkv

using namespace tkv;

extern "C" int tkv_pack_codes(const uint8_t* codes, uint8_t* packed, int64_t rows, int D, int nbits,
                              void* stream) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(rows >= 0 && D > 0, TKV_ERR_INVALID, "pack_codes: bad sizes rows=%lld D=%d",
              (long long)rows, D);
  const int P = 8 / nbits;
  TKV_REQUIRE(D % P == 0, TKV_ERR_INVALID, "head_dim %d must be divisible by %d for %d-bit packing",
              D, P, nbits);
  const int64_t n = rows * (D / P);
  if (n == 0) return TKV_OK;  // an empty tensor has no storage: nothing to check, nothing to do
  TKV_REQUIRE(codes && packed, TKV_ERR_INVALID, "pack_codes: null pointer");
  TKV_REQUIRE((n + 255) / 256 <= 0x7fffffffLL, TKV_ERR_INVALID, "pack_codes: tensor too large");
  if ((D / P) % 8 == 0 && ((uintptr_t)codes & 7u) == 0 && ((uintptr_t)packed & 7u) == 0) {
    const int64_t nt = n / 8;
    const int blocks8 = (int)((nt + kItemsPerThread * 256 - 1) / (kItemsPerThread * 256));
    if (nbits == 4)
      pack_codes8_kernel<4><<<blocks8, 256, 0, (cudaStream_t)stream>>>(codes, packed, nt, D);
    else
      pack_codes8_kernel<2><<<blocks8, 256, 0, (cudaStream_t)stream>>>(codes, packed, nt, D);
    TKV_CUDA(cudaGetLastError());
    return TKV_OK;
  }
  const int blocks = (int)((n + 255) / 256);
  if (nbits == 4)
    pack_codes_kernel<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(codes, packed, n, D);
  else
    pack_codes_kernel<2><<<blocks, 256, 0, (cudaStream_t)stream>>>(codes, packed, n, D);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}

extern "C" int tkv_unpack_codes(const uint8_t* packed, uint8_t* codes, int64_t rows, int D,
                                int nbits, void* stream) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(rows >= 0 && D > 0, TKV_ERR_INVALID, "unpack_codes: bad sizes rows=%lld D=%d",
              (long long)rows, D);
  const int P = 8 / nbits;
  TKV_REQUIRE(D % P == 0, TKV_ERR_INVALID, "head_dim %d must be divisible by %d", D, P);
  const int64_t n = rows * D;
  if (n == 0) return TKV_OK;
  TKV_REQUIRE(codes && packed, TKV_ERR_INVALID, "unpack_codes: null pointer");
  TKV_REQUIRE((n + 255) / 256 <= 0x7fffffffLL, TKV_ERR_INVALID, "unpack_codes: tensor too large");
  if ((D / P) % 8 == 0 && ((uintptr_t)codes & 7u) == 0 && ((uintptr_t)packed & 7u) == 0) {
    const int64_t nt = rows * (D / P / 8);
    const int blocks8 = (int)((nt + kItemsPerThread * 256 - 1) / (kItemsPerThread * 256));
    if (nbits == 4)
      unpack_codes8_kernel<4><<<blocks8, 256, 0, (cudaStream_t)stream>>>(packed, codes, nt, D);
    else
      unpack_codes8_kernel<2><<<blocks8, 256, 0, (cudaStream_t)stream>>>(packed, codes, nt, D);
    TKV_CUDA(cudaGetLastError());
    return TKV_OK;
  }
  const int blocks = (int)((n + 255) / 256);
  if (nbits == 4)
    unpack_codes_kernel<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, codes, n, D);
  else
    unpack_codes_kernel<2><<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, codes, n, D);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}

namespace {
inline int log2i(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

template <typename T, int E>
int launch_quantize_e(const void* x, uint8_t* packed, void* scale, void* zero, int64_t rows, int D,
                      int nbits, int gs, cudaStream_t stream, const AppendMap& am) {
  const int tpr_shift = log2i(D / E), lpg_shift = log2i(gs / E);  // powers of two, checked by the caller
  const int rows_per_block = kRowsPerThread * (256 >> tpr_shift);
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  TKV_REQUIRE(blocks <= 0x7fffffffLL, TKV_ERR_INVALID, "quantize_pack: tensor too large");
  if (nbits == 4)
    quantize_pack_kernel<T, 4, E><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, rows, tpr_shift, lpg_shift, am);
  else
    quantize_pack_kernel<T, 2, E><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, rows, tpr_shift, lpg_shift, am);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}

template <typename T>
int launch_quantize(const void* x, uint8_t* packed, void* scale, void* zero, int64_t rows, int D,
                    int nbits, int gs, cudaStream_t stream, const AppendMap am = AppendMap{}) {
  // 16 elements per thread where a 16-bit row gives every bit slice and every group a whole thread
  if constexpr (!std::is_same<T, float>::value) {
    if (gs >= 16 && D / 16 >= 8 / nbits && ((uintptr_t)packed & 15u) == 0)
      return launch_quantize_e<T, 16>(x, packed, scale, zero, rows, D, nbits, gs, stream, am);
  }
  return launch_quantize_e<T, 8>(x, packed, scale, zero, rows, D, nbits, gs, stream, am);
}
}  // namespace

extern "C" int tkv_quantize_pack(const void* x, int in_dtype, uint8_t* packed, void* scale,
                                 void* zero, int64_t rows, int D, int nbits, int gs, void* stream) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(rows >= 0, TKV_ERR_INVALID, "quantize_pack: rows=%lld", (long long)rows);
  TKV_REQUIRE(gs > 0 && D > 0 && D % gs == 0, TKV_ERR_INVALID,
              "group_size %d must divide head_dim %d", gs, D);
  if (rows == 0) return TKV_OK;  // an empty tensor has no storage: nothing to check, nothing to do
  TKV_REQUIRE(x && packed && scale && zero, TKV_ERR_INVALID, "quantize_pack: null pointer");
  // One thread owns 8 elements; a row (<= 256 elements) and a group must map to
  // whole, aligned lane ranges of one warp.
  TKV_REQUIRE(pow2(D) && D >= 16 && D <= 256 && pow2(gs) && gs >= 8, TKV_ERR_UNSUPPORTED,
              "quantize_pack: built for power-of-two head_dim in [16, 256] and power-of-two "
              "group_size >= 8 (got head_dim=%d, group_size=%d)", D, gs);
  TKV_REQUIRE((D * nbits / 8) % 8 == 0, TKV_ERR_UNSUPPORTED,
              "quantize_pack: packed row of %d bytes is not a multiple of 8", D * nbits / 8);
  TKV_REQUIRE(aligned16(x) && ((uintptr_t)packed & 7u) == 0, TKV_ERR_ALIGN,
              "quantize_pack: x must be 16-byte and packed 8-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  switch (in_dtype) {
    case TKV_DTYPE_F16: return launch_quantize<__half>(x, packed, scale, zero, rows, D, nbits, gs, s);
    case TKV_DTYPE_BF16: return launch_quantize<__nv_bfloat16>(x, packed, scale, zero, rows, D, nbits, gs, s);
    case TKV_DTYPE_F32: return launch_quantize<float>(x, packed, scale, zero, rows, D, nbits, gs, s);
  }
  set_error("quantize_pack: bad dtype %d", in_dtype);
  return TKV_ERR_INVALID;
}

static int check_quantize_shape(const char* who, int D, int nbits, int gs) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(gs > 0 && D > 0 && D % gs == 0, TKV_ERR_INVALID,
              "group_size %d must divide head_dim %d", gs, D);
  TKV_REQUIRE(pow2(D) && D >= 16 && D <= 256 && pow2(gs) && gs >= 8, TKV_ERR_UNSUPPORTED,
              "%s: built for power-of-two head_dim in [16, 256] and power-of-two "
              "group_size >= 8 (got head_dim=%d, group_size=%d)", who, D, gs);
  TKV_REQUIRE((D * nbits / 8) % 8 == 0, TKV_ERR_UNSUPPORTED,
              "%s: packed row of %d bytes is not a multiple of 8", who, D * nbits / 8);
  return TKV_OK;
}

extern "C" int tkv_quantize_append(const void* x, int in_dtype, uint8_t* packed, void* scale,
                                   void* zero, int B, int HKV, int T_new, int64_t S_cap, int D,
                                   int nbits, int gs, const int32_t* positions, int pos0,
                                   void* stream) {
  TKV_REQUIRE((x || T_new == 0) && packed && scale && zero, TKV_ERR_INVALID,
              "quantize_append: null pointer");
  TKV_REQUIRE(B > 0 && HKV > 0 && T_new >= 0 && S_cap > 0, TKV_ERR_INVALID,
              "quantize_append: bad sizes B=%d HKV=%d T_new=%d S_cap=%lld", B, HKV, T_new,
              (long long)S_cap);
  int rc = check_quantize_shape("quantize_append", D, nbits, gs);
  if (rc != TKV_OK) return rc;
  TKV_REQUIRE(aligned16(x) && ((uintptr_t)packed & 7u) == 0, TKV_ERR_ALIGN,
              "quantize_append: x must be 16-byte and packed 8-byte aligned");
  TKV_REQUIRE(positions != nullptr || (pos0 >= 0 && (int64_t)pos0 + T_new <= S_cap), TKV_ERR_INVALID,
              "quantize_append: tokens [%d, %d) do not fit a cache of %lld rows", pos0, pos0 + T_new,
              (long long)S_cap);
  if (T_new == 0) return TKV_OK;
  TKV_REQUIRE((int64_t)B * HKV < (1LL << 31), TKV_ERR_INVALID,
              "quantize_append: B*HKV = %lld sequences x heads exceed 2^31", (long long)B * HKV);
  AppendMap am{positions, pos0, T_new, HKV, S_cap};
  const int64_t rows = (int64_t)B * HKV * T_new;
  cudaStream_t s = (cudaStream_t)stream;
  switch (in_dtype) {
    case TKV_DTYPE_F16: return launch_quantize<__half>(x, packed, scale, zero, rows, D, nbits, gs, s, am);
    case TKV_DTYPE_BF16: return launch_quantize<__nv_bfloat16>(x, packed, scale, zero, rows, D, nbits, gs, s, am);
    case TKV_DTYPE_F32: return launch_quantize<float>(x, packed, scale, zero, rows, D, nbits, gs, s, am);
  }
  set_error("quantize_append: bad dtype %d", in_dtype);
  return TKV_ERR_INVALID;
}

namespace {
template <typename T>
int launch_dequant(const uint8_t* packed, const void* scale, const void* zero, void* out,
                   int64_t rows, int D, int nbits, int gs, cudaStream_t stream) {
  const int64_t n = rows * D;
  const int64_t blocks = (n + 255) / 256;
  TKV_REQUIRE(blocks <= 0x7fffffffLL, TKV_ERR_INVALID, "dequantize: tensor too large");
  const int DP = D / (8 / nbits);
  if (DP % 8 == 0 && gs % 8 == 0 && ((uintptr_t)packed & 7u) == 0 && aligned16(out)) {
    const int64_t nt = rows * (DP / 8);
    const int blocks8 = (int)((nt + kItemsPerThread * 256 - 1) / (kItemsPerThread * 256));
    if (nbits == 4)
      dequantize8_kernel<T, 4><<<blocks8, 256, 0, stream>>>(packed, (const __half*)scale,
                                                            (const __half*)zero, (T*)out, nt, D, gs);
    else
      dequantize8_kernel<T, 2><<<blocks8, 256, 0, stream>>>(packed, (const __half*)scale,
                                                            (const __half*)zero, (T*)out, nt, D, gs);
    TKV_CUDA(cudaGetLastError());
    return TKV_OK;
  }
  if (nbits == 4)
    dequantize_kernel<T, 4><<<(int)blocks, 256, 0, stream>>>(packed, (const __half*)scale,
                                                             (const __half*)zero, (T*)out, n, D, gs);
  else
    dequantize_kernel<T, 2><<<(int)blocks, 256, 0, stream>>>(packed, (const __half*)scale,
                                                             (const __half*)zero, (T*)out, n, D, gs);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}
}  // namespace

extern "C" int tkv_dequantize(const uint8_t* packed, const void* scale, const void* zero, void* out,
                              int out_dtype, int64_t rows, int D, int nbits, int gs, void* stream) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(rows >= 0, TKV_ERR_INVALID, "dequantize: rows=%lld", (long long)rows);
  TKV_REQUIRE(gs > 0 && D > 0 && D % gs == 0 && D % (8 / nbits) == 0, TKV_ERR_INVALID,
              "dequantize: group_size %d must divide head_dim %d", gs, D);
  if (rows == 0) return TKV_OK;
  TKV_REQUIRE(packed && scale && zero && out, TKV_ERR_INVALID, "dequantize: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  switch (out_dtype) {
    case TKV_DTYPE_F16: return launch_dequant<__half>(packed, scale, zero, out, rows, D, nbits, gs, s);
    case TKV_DTYPE_BF16: return launch_dequant<__nv_bfloat16>(packed, scale, zero, out, rows, D, nbits, gs, s);
    case TKV_DTYPE_F32: return launch_dequant<float>(packed, scale, zero, out, rows, D, nbits, gs, s);
  }
  set_error("dequantize: bad dtype %d", out_dtype);
  return TKV_ERR_INVALID;
}

namespace {
template <typename T>
int launch_keys_channel(const void* x, uint8_t* packed, void* scale, void* zero, int64_t BH, int64_t S,
                        int64_t S_q, int D, int nbits, cudaStream_t stream) {
  const int64_t n_blocks = BH * (S_q / tkv::kChanTok);
  const int per_cta = 512 / D;  // token blocks per CTA of 256 threads
  const int64_t blocks = (n_blocks + per_cta - 1) / per_cta;
  TKV_REQUIRE(blocks <= 0x7fffffffLL, TKV_ERR_INVALID, "quantize_keys_per_channel: tensor too large");
  if (nbits == 4)
    tkv::quantize_keys_channel_kernel<T, 4><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, S, S_q, D, n_blocks);
  else
    tkv::quantize_keys_channel_kernel<T, 2><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, S, S_q, D, n_blocks);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}
}  // namespace

extern "C" int tkv_quantize_keys_per_channel(const void* x, int in_dtype, uint8_t* packed, void* scale,
                                             void* zero, int64_t BH, int64_t S, int64_t S_q, int D,
                                             int nbits, void* stream) {
  TKV_REQUIRE(nbits == 2 || nbits == 4, TKV_ERR_INVALID, "nbits must be one of (2, 4), got %d", nbits);
  TKV_REQUIRE(BH >= 0 && S >= 0 && S_q >= 0 && S_q <= S && S_q % tkv::kChanTok == 0, TKV_ERR_INVALID,
              "quantize_keys_per_channel: the quantised part (%lld of %lld tokens) must be a multiple of "
              "%d tokens", (long long)S_q, (long long)S, tkv::kChanTok);
  TKV_REQUIRE(pow2(D) && D >= 32 && D <= 256, TKV_ERR_UNSUPPORTED,
              "quantize_keys_per_channel: built for power-of-two head_dim in [32, 256], got %d", D);
  if (BH == 0 || S_q == 0) return TKV_OK;
  TKV_REQUIRE(x && packed && scale && zero, TKV_ERR_INVALID, "quantize_keys_per_channel: null pointer");
  TKV_REQUIRE(D * nbits / 8 >= 16, TKV_ERR_UNSUPPORTED,
              "quantize_keys_per_channel: packed rows of %d bytes are shorter than 16", D * nbits / 8);
  TKV_REQUIRE(aligned16(packed) && ((uintptr_t)x & 7u) == 0 && ((uintptr_t)scale & 3u) == 0 &&
                  ((uintptr_t)zero & 3u) == 0,
              TKV_ERR_ALIGN, "quantize_keys_per_channel: packed must be 16-byte, x 8-byte, scale and zero 4-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  switch (in_dtype) {
    case TKV_DTYPE_F16: return launch_keys_channel<__half>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
    case TKV_DTYPE_BF16: return launch_keys_channel<__nv_bfloat16>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
    case TKV_DTYPE_F32: return launch_keys_channel<float>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
  }
  set_error("quantize_keys_per_channel: bad dtype %d", in_dtype);
  return TKV_ERR_INVALID;
}
