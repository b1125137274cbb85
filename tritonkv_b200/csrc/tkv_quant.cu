// Group-wise quantiser and split-P packing kernels (sm_100a).
//
// Replaces the eager PyTorch chain of the reference's quantize.py with one launch
// each: pack_codes (:149-169), unpack_codes (:172-183), quantize_groupwise (:186-236),
// dequantize_groupwise (:239-246).  Integer and rounding behaviour is bit-exact:
// every float operation below is a single IEEE round-to-nearest operation written
// with an explicit intrinsic so that neither FMA contraction nor a fast-math flag
// can change it.
#include "tkv_common.cuh"

namespace tkv {

// ---------------------------------------------------------------- quantize + pack
// Each thread owns 8 consecutive elements of a row.  A quantisation group spans
// GS/8 adjacent lanes; min/max are butterfly-reduced inside it.  The 8 codes of a
// thread form a 64-bit word (one code per byte); split-P packing ORs the words of
// the P lanes that hold dims j, j+DP, ... shifted by their bit-slice position.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]);

template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// Where the rows go when new tokens are appended to a preallocated cache (cap == 0: in place).
struct AppendMap {
  const int32_t* pos;  // per-sequence first free slot, or null for pos0 everywhere
  int pos0;
  int t_new;           // new tokens per (sequence, head)
  int hkv;             // heads per sequence
  int64_t cap;         // token rows per (sequence, head) in the cache
};

template <typename T, int NBITS>
__global__ void __launch_bounds__(256)
    quantize_pack_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed,
                         __half* __restrict__ scale, __half* __restrict__ zero, int64_t rows,
                         int D, int gs, const AppendMap am) {
  constexpr int P = 8 / NBITS;
  constexpr float QMAX = float((1 << NBITS) - 1);
  const int tpr = D >> 3;                 // threads per row
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = tid / tpr;
  const int c = (int)(tid % tpr);         // 8-element column block
  const bool live = row < rows;
  // Lanes past the end mirror the last row so the shuffles below stay full-warp.
  const int64_t r = live ? row : rows - 1;

  float v[8];
  load8<T>(x + r * D + 8 * c, v);
  float mn = v[0], mx = v[0];
  bool has_nan = v[0] != v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    mn = fminf(mn, v[i]);
    mx = fmaxf(mx, v[i]);
    has_nan |= v[i] != v[i];
  }
  const int lanes_per_group = gs >> 3;
  for (int off = 1; off < lanes_per_group; off <<= 1) {
    mn = fminf(mn, __shfl_xor_sync(kFullMask, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, off));
    has_nan |= __shfl_xor_sync(kFullMask, (int)has_nan, off) != 0;
  }
  // torch's amin/amax propagate NaN where fminf/fmaxf drop it: a group that holds a NaN
  // gets zero = NaN, scale = 1 and all codes 0, as the reference produces.
  if (has_nan) mn = mx = __int_as_float(0x7fc00000);
  float sc = __fdiv_rn(__fsub_rn(mx, mn), QMAX);
  sc = (sc > 0.f) ? sc : 1.f;
  const __half sc16 = __float2half_rn(sc);
  const __half ze16 = __float2half_rn(mn);
  const float scf = __half2float(sc16), zef = __half2float(ze16);

  uint64_t word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float t = rintf(__fdiv_rn(__fsub_rn(v[i], zef), scf));
    t = fminf(fmaxf(t, 0.f), QMAX);
    word |= (uint64_t)(uint32_t)(int)t << (8 * i);
  }
  // split-P: lane c = p*TPS + c' contributes bit slice p of bytes [8c', 8c'+8)
  const int tps = tpr / P;
  const int p = c / tps;
  word <<= (NBITS * p);
  for (int off = tps; off < tpr; off <<= 1) {
    const uint32_t lo = __shfl_xor_sync(kFullMask, (uint32_t)word, off);
    const uint32_t hi = __shfl_xor_sync(kFullMask, (uint32_t)(word >> 32), off);
    word |= ((uint64_t)hi << 32) | lo;
  }
  // Output row: the input row itself, or (append) slot pos[b] + t of sequence (b, head)
  // in a cache of `cap` token rows per sequence; tokens that fall outside are dropped.
  int64_t orow = row;
  bool keep = live;
  if (am.cap > 0 && live) {
    const int64_t bh = row / am.t_new;
    const int t = (int)(row - bh * am.t_new);
    const int64_t at = (am.pos ? (int64_t)am.pos[bh / am.hkv] : (int64_t)am.pos0) + t;
    keep = at >= 0 && at < am.cap;
    orow = bh * am.cap + at;
  }
  if (keep) {
    if (p == 0) *reinterpret_cast<uint64_t*>(packed + orow * (D / P) + 8 * c) = word;
    if ((c % lanes_per_group) == 0) {
      const int64_t gi = orow * (D / gs) + (8 * c) / gs;
      scale[gi] = sc16;
      zero[gi] = ze16;
    }
  }
}

// ---------------------------------------------------------------- per-channel keys
// Keys quantised per channel: a group is kChanTok consecutive tokens of ONE head dimension
// (the reference describes the format as future work, docs/future_work.md:229-293, and has
// no implementation of it).  Same per-element arithmetic as quantize_pack_kernel on the other
// axis; the codes keep the split-P byte layout along the head dimension, scale and zero are
// one row of D values per block of kChanTok tokens.
// One CTA per (sequence x head, token block), one thread per head dimension: the thread walks
// the block's tokens of its dimension (the loads of a warp are one contiguous row piece),
// derives scale/zero, leaves its codes in shared memory, and the CTA then packs whole rows.
constexpr int kChanTok = 32;

template <typename T>
__device__ __forceinline__ float load1(const T* p) { return (float)*p; }
template <>
__device__ __forceinline__ float load1<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

template <typename T, int NBITS>
__global__ void __launch_bounds__(256)
    quantize_keys_channel_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed,
                                 __half* __restrict__ scale, __half* __restrict__ zero,
                                 int64_t S, int64_t S_q, int D) {
  constexpr int P = 8 / NBITS;
  constexpr float QMAX = float((1 << NBITS) - 1);
  __shared__ uint8_t codes[kChanTok][256];
  const int d = threadIdx.x;
  const int64_t blocks_per_seq = S_q / kChanTok;
  const int64_t bh = blockIdx.x / blocks_per_seq, tb = blockIdx.x - bh * blocks_per_seq;
  const T* src = x + (bh * S + tb * kChanTok) * D + d;
  float v[kChanTok];
  float mn, mx;
  bool has_nan = false;
#pragma unroll
  for (int t = 0; t < kChanTok; ++t) {
    v[t] = load1<T>(src + (int64_t)t * D);
    has_nan |= v[t] != v[t];
    mn = t == 0 ? v[0] : fminf(mn, v[t]);
    mx = t == 0 ? v[0] : fmaxf(mx, v[t]);
  }
  if (has_nan) mn = mx = __int_as_float(0x7fc00000);  // NaN propagates, as in the per-token quantiser
  float sc = __fdiv_rn(__fsub_rn(mx, mn), QMAX);
  sc = (sc > 0.f) ? sc : 1.f;
  const __half sc16 = __float2half_rn(sc), ze16 = __float2half_rn(mn);
  const float scf = __half2float(sc16), zef = __half2float(ze16);
  const int64_t mrow = (bh * blocks_per_seq + tb) * D + d;
  scale[mrow] = sc16;
  zero[mrow] = ze16;
#pragma unroll
  for (int t = 0; t < kChanTok; ++t) {
    float c = rintf(__fdiv_rn(__fsub_rn(v[t], zef), scf));
    c = fminf(fmaxf(c, 0.f), QMAX);
    codes[t][d] = (uint8_t)(int)c;
  }
  __syncthreads();
  // pack: byte j of a token = OR_p code[j + p*DP] << (p*NBITS); D threads write kChanTok*DP bytes
  const int DP = D / P;
  for (int i = threadIdx.x; i < kChanTok * DP; i += blockDim.x) {
    const int t = i / DP, j = i - t * DP;
    uint32_t b = 0;
#pragma unroll
    for (int p = 0; p < P; ++p) b |= (uint32_t)codes[t][j + p * DP] << (p * NBITS);
    packed[((bh * S_q) + tb * kChanTok + t) * DP + j] = (uint8_t)b;
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
  const int blocks = (int)((n + 255) / 256);
  if (nbits == 4)
    unpack_codes_kernel<4><<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, codes, n, D);
  else
    unpack_codes_kernel<2><<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, codes, n, D);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
}

namespace {
template <typename T>
int launch_quantize(const void* x, uint8_t* packed, void* scale, void* zero, int64_t rows, int D,
                    int nbits, int gs, cudaStream_t stream, const AppendMap am = AppendMap{}) {
  const int64_t threads = rows * (D / 8);
  const int64_t blocks = (threads + 255) / 256;
  TKV_REQUIRE(blocks <= 0x7fffffffLL, TKV_ERR_INVALID, "quantize_pack: tensor too large");
  if (nbits == 4)
    quantize_pack_kernel<T, 4><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, rows, D, gs, am);
  else
    quantize_pack_kernel<T, 2><<<(int)blocks, 256, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, rows, D, gs, am);
  TKV_CUDA(cudaGetLastError());
  return TKV_OK;
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
  const int64_t blocks = BH * (S_q / tkv::kChanTok);
  TKV_REQUIRE(blocks <= 0x7fffffffLL, TKV_ERR_INVALID, "quantize_keys_per_channel: tensor too large");
  if (nbits == 4)
    tkv::quantize_keys_channel_kernel<T, 4><<<(int)blocks, D, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, S, S_q, D);
  else
    tkv::quantize_keys_channel_kernel<T, 2><<<(int)blocks, D, 0, stream>>>(
        (const T*)x, packed, (__half*)scale, (__half*)zero, S, S_q, D);
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
  cudaStream_t s = (cudaStream_t)stream;
  switch (in_dtype) {
    case TKV_DTYPE_F16: return launch_keys_channel<__half>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
    case TKV_DTYPE_BF16: return launch_keys_channel<__nv_bfloat16>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
    case TKV_DTYPE_F32: return launch_keys_channel<float>(x, packed, scale, zero, BH, S, S_q, D, nbits, s);
  }
  set_error("quantize_keys_per_channel: bad dtype %d", in_dtype);
  return TKV_ERR_INVALID;
}
