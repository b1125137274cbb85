// Log-sum-exp merge of split-K partials (sm_100a).
//
// Replaces _combine_splits of the reference (kernels/fused_decode_attn.py:355-395):
//     out = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),   M = max_s m_s
// The reference walks the splits sequentially in one program per (batch, head); with
// a device-filling split count (hundreds at batch 1) that loop is a chain of
// dependent L2 round trips.  Here one CTA of 256 threads owns a (batch, head, 32-dim
// slice): the maximum is a block reduction, then 32 thread groups each take every
// 32nd split with independent float4 loads, and the groups are summed through warp
// shuffles and shared memory.  Splits with m = -inf (empty) weigh zero.
// With out_m/out_l given, the merged partial is written unnormalised together with
// (M, L): the wire format of a cross-GPU history split.
#include "tkv_split_common.cuh"

namespace tkv {

constexpr int kCombineThreads = 256;
constexpr int kCombineSlice = 32;  // head dims per CTA

// What thread `tid` < 8 of a CTA holds after the block-wide merge of one (row, 32-dim slice).
struct CombineResult {
  float4 r;  // unnormalised sum_s acc_s 2^(m_s - M), dims d0 + 4 tid .. +3
  float M;   // max_s m_s
  float L;   // sum_s l_s 2^(m_s - M)
};

__device__ __forceinline__ CombineResult combine_reduce(const float* __restrict__ acc,
                                                        const float* __restrict__ m,
                                                        const float* __restrict__ l, int NS,
                                                        int64_t a_row, int64_t a_slot,
                                                        int64_t ml_row, int64_t ml_slot, int row,
                                                        int d0) {
  CombineResult res;
  res.r = make_float4(0.f, 0.f, 0.f, 0.f);
  res.L = 0.f;
  __shared__ float red_m[8];
  __shared__ float4 red_a[8][8];
  __shared__ float red_l[8];
  __shared__ float sh_m[kCombineThreads];
  __shared__ float sh_l[kCombineThreads];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sg = tid >> 3, dl = tid & 7; // split group (0..31), float4 index inside the slice
  const float* mrow = m + (int64_t)row * ml_row;
  const float* lrow = l + (int64_t)row * ml_row;
  const float* arow = acc + (int64_t)row * a_row + d0 + dl * 4;

  constexpr int kCached = 8;  // slots per thread kept in registers: NS <= 256
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  float L = 0.f;
  float M;
  if (NS <= 32 * kCached) {
    // One round trip: every load is issued before any value is used.  The acc rows go
    // straight to registers; (m, l) of slot `tid` are fetched once per CTA and shared
    // through shared memory instead of 16 scalar loads per thread.  Loads bypass L1
    // (each value is read once; measured 0.2 us faster than the read-only path).
    float4 xs[kCached];
#pragma unroll
    for (int i = 0; i < kCached; ++i) {
      const int s = min(sg + 32 * i, NS - 1);  // slots past NS re-read the last one, unused
      xs[i] = __ldcg(reinterpret_cast<const float4*>(arow + (int64_t)s * a_slot));
    }
    const int sm = min(tid, NS - 1);
    float mloc = __ldcg(mrow + sm * ml_slot);
    const float lmine = __ldcg(lrow + sm * ml_slot);
    if (tid >= NS) mloc = -INFINITY;
    sh_m[tid] = mloc;
    sh_l[tid] = lmine;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
      mloc = fmaxf(mloc, __shfl_xor_sync(kFullMask, mloc, off));
    if (lane == 0) red_m[warp] = mloc;
    __syncthreads();
    M = red_m[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) M = fmaxf(M, red_m[w]);
#pragma unroll
    for (int i = 0; i < kCached; ++i) {
      const float ms = sh_m[sg + 32 * i];  // -inf past NS and for empty slots
      if (ms > -INFINITY) {  // empty slots (m = -inf) may hold anything in acc: never use it
        const float w = ex2(ms - M);
        a.x = fmaf(w, xs[i].x, a.x);
        a.y = fmaf(w, xs[i].y, a.y);
        a.z = fmaf(w, xs[i].z, a.z);
        a.w = fmaf(w, xs[i].w, a.w);
        L = fmaf(w, sh_l[sg + 32 * i], L);
      }
    }
  } else {
    float mloc = -INFINITY;
    for (int s = tid; s < NS; s += kCombineThreads) mloc = fmaxf(mloc, __ldcg(mrow + s * ml_slot));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
      mloc = fmaxf(mloc, __shfl_xor_sync(kFullMask, mloc, off));
    if (lane == 0) red_m[warp] = mloc;
    __syncthreads();
    M = red_m[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) M = fmaxf(M, red_m[w]);
#pragma unroll 4
    for (int s = sg; s < NS; s += 32) {
      const float ms = __ldcg(mrow + s * ml_slot);
      if (ms > -INFINITY) {
        const float w = ex2(ms - M);
        const float4 x = __ldcg(reinterpret_cast<const float4*>(arow + (int64_t)s * a_slot));
        a.x = fmaf(w, x.x, a.x);
        a.y = fmaf(w, x.y, a.y);
        a.z = fmaf(w, x.z, a.z);
        a.w = fmaf(w, x.w, a.w);
        L = fmaf(w, __ldcg(lrow + s * ml_slot), L);
      }
    }
  }
  // the 4 split groups of a warp (lanes dl, dl+8, dl+16, dl+24)
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
    a.x += __shfl_xor_sync(kFullMask, a.x, off);
    a.y += __shfl_xor_sync(kFullMask, a.y, off);
    a.z += __shfl_xor_sync(kFullMask, a.z, off);
    a.w += __shfl_xor_sync(kFullMask, a.w, off);
    L += __shfl_xor_sync(kFullMask, L, off);
  }
  if (lane < 8) red_a[warp][lane] = a;
  if (lane == 0) red_l[warp] = L;
  __syncthreads();
  if (tid < 8) {
    float4 r = red_a[0][tid];
    float Lt = red_l[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      const float4 x = red_a[w][tid];
      r.x += x.x;
      r.y += x.y;
      r.z += x.z;
      r.w += x.w;
      Lt += red_l[w];
    }
    res.r = r;
    res.L = Lt;
  }
  res.M = M;
  return res;
}

__global__ void __launch_bounds__(kCombineThreads)
    combine_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                   const float* __restrict__ l, float* __restrict__ out, float* __restrict__ out_m,
                   float* __restrict__ out_l, int NS, int D, int64_t a_row, int64_t a_slot,
                   int64_t ml_row, int64_t ml_slot) {
  const int tid = threadIdx.x;
  const int row = blockIdx.x;  // b*HQ + h
  const int d0 = blockIdx.y * kCombineSlice;
  pdl_launch_dependents();  // the next kernel of the stream may start its prologue
  pdl_wait();               // partials come from the kernel launched just before this one
  const CombineResult c = combine_reduce(acc, m, l, NS, a_row, a_slot, ml_row, ml_slot, row, d0);
  if (tid < 8) {
    float4 r = c.r;
    if (out_m == nullptr) {
      const float inv = c.L > 0.f ? 1.f / c.L : 0.f;
      r.x *= inv;
      r.y *= inv;
      r.z *= inv;
      r.w *= inv;
    } else if (tid == 0 && blockIdx.y == 0) {
      out_m[row] = c.M;
      out_l[row] = c.L;
    }
    *reinterpret_cast<float4*>(out + (int64_t)row * D + d0 + tid * 4) = r;
  }
}

// ---------------------------------------------------------------------------------
// Cross-GPU exchange of one merged partial per head over peer memory (history split).
//
// Every rank owns a receive buffer of 2 x world blocks, mapped on every peer.  A block is
// the wire layout [acc rows*D | m rows | l rows] with every float widened to the 8-byte
// pair {value, step}: an 8-byte store is delivered whole, so the step number that rides
// with each value tells the reader that THIS value has arrived -- no fence, no flag, no
// acknowledgement on the path, one NVLink latency (a fenced data-then-flag version of
// this exchange cost three).  push merges the local split partials like combine_kernel
// and stores the result into block (step parity, own rank) of EVERY rank's buffer.
// wait-merge reads the world blocks of this step, each thread polling its own pairs until
// they carry the step (bounded; on expiry it records a status and goes on), merges them,
// and every CTA bumps the step counter of its (row, slice) in local memory.  Two
// parities suffice: a rank can only be one step ahead of the slowest, because each step
// consumes every rank's block.
constexpr int kMaxPeers = 8;
struct Exchange {
  uint2* data[kMaxPeers];  // rank j's receive buffer, as mapped in this process
  uint32_t* state;         // this rank's step counters, one per (row, 32-dim slice), local memory
  int world, rank, rows, wire;  // wire = pairs per block
};

__device__ int g_exchange_status;  // 0 ok, 1 a bounded wait for a peer's data gave up

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// A {value, step} pair moves as ONE 64-bit access: the memory model gives single-copy
// atomicity to an aligned 8-byte scalar access, not to the two halves of a vector access,
// and the protocol needs the step never to be seen without its value.
__device__ __forceinline__ uint2 ld_volatile_pair(const uint2* p) {
  uint64_t w;
  asm volatile("ld.volatile.global.u64 %0, [%1];\n" : "=l"(w) : "l"(p) : "memory");
  uint2 v;
  asm("mov.b64 {%0,%1}, %2;\n" : "=r"(v.x), "=r"(v.y) : "l"(w));
  return v;
}
__device__ __forceinline__ void st_volatile_pair(uint2* p, float x, uint32_t step) {
  uint64_t w;
  asm("mov.b64 %0, {%1,%2};\n" : "=l"(w) : "r"(__float_as_uint(x)), "r"(step));
  asm volatile("st.volatile.global.u64 [%0], %1;\n" ::"l"(p), "l"(w) : "memory");
}

// Cross-rank half of the exchange for one (row, 32-dim slice): warp j reads rank j's block of
// this step, lane = dim inside the slice, polling (bounded) until each pair carries the
// step; then the log-sum-exp merge, the store of the normalised output, and the ticket that
// lets the last CTA of the grid bump the step.
__device__ __forceinline__ void wait_merge_store(float* __restrict__ out, int D, const Exchange& ex,
                                                 uint32_t step, int row, int d0) {
  __shared__ float sh_x[kMaxPeers][kCombineSlice];
  __shared__ float sh_ml[kMaxPeers][2];
  const int tid = threadIdx.x, j = tid >> 5, lane = tid & 31;
  if (j < ex.world) {
    const uint2* src = ex.data[ex.rank] + (int64_t)((step & 1) * ex.world + j) * ex.wire;
    const uint2* px = src + (int64_t)row * D + d0 + lane;
    // lanes 0 and 1 also fetch (m, l) of the row
    const uint2* pml = src + (int64_t)ex.rows * D + (lane == 1 ? ex.rows : 0) + row;
    uint2 x = ld_volatile_pair(px);
    uint2 ml = lane < 2 ? ld_volatile_pair(pml) : make_uint2(0u, step);
    int polls = 0;
    while (x.y != step || ml.y != step) {
      if (++polls > (1 << 18)) {  // a few tenths of a second with the pause below: a peer is gone
        atomicExch(&g_exchange_status, 1);
        break;
      }
      __nanosleep(100);
      if (x.y != step) x = ld_volatile_pair(px);
      if (ml.y != step) ml = ld_volatile_pair(pml);
    }
    sh_x[j][lane] = __uint_as_float(x.x);
    if (lane < 2) sh_ml[j][lane] = __uint_as_float(ml.x);
  }
  __syncthreads();
  if (tid < kCombineSlice) {
    float M = -INFINITY;
    for (int r = 0; r < ex.world; ++r) M = fmaxf(M, sh_ml[r][0]);
    float a = 0.f, L = 0.f;
    for (int r = 0; r < ex.world; ++r) {
      const float mr = sh_ml[r][0];
      if (mr > -INFINITY) {  // a rank without tokens sends m = -inf
        const float w = ex2(mr - M);
        a = fmaf(w, sh_x[r][tid], a);
        L = fmaf(w, sh_ml[r][1], L);
      }
    }
    out[(int64_t)row * D + d0 + tid] = L > 0.f ? a / L : 0.f;
  }
  // this CTA's step counter (local memory; only the CTA of the same (row, slice) of the next
  // exchange reads it, and that grid follows this one in the stream): a plain store, so the
  // kernel does not end on the round trip of an atomic ticket
  if (tid == 0) ex.state[blockIdx.x * gridDim.y + blockIdx.y] = step;
}

// Stores the merged (row, slice) of this rank, tagged with the step, into block
// (step parity, own rank) of every rank's receive buffer.  Threads 0..7 hold the result.
__device__ __forceinline__ void push_to_peers(const CombineResult& c, const Exchange& ex, uint32_t step,
                                              int D, int row, int d0, bool first_slice) {
  const int tid = threadIdx.x;
  if (tid < 8) {
    const int64_t blk = (int64_t)((step & 1) * ex.world + ex.rank) * ex.wire;
    const int64_t e = (int64_t)row * D + d0 + tid * 4;
    for (int j = 0; j < ex.world; ++j) {
      uint2* dst = ex.data[j] + blk;
      st_volatile_pair(dst + e, c.r.x, step);
      st_volatile_pair(dst + e + 1, c.r.y, step);
      st_volatile_pair(dst + e + 2, c.r.z, step);
      st_volatile_pair(dst + e + 3, c.r.w, step);
      if (tid == 0 && first_slice) {
        st_volatile_pair(dst + (int64_t)ex.rows * D + row, c.M, step);
        st_volatile_pair(dst + (int64_t)ex.rows * D + ex.rows + row, c.L, step);
      }
    }
  }
}

__global__ void __launch_bounds__(kCombineThreads)
    combine_push_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                        const float* __restrict__ l, int NS, int D, int64_t a_row, int64_t a_slot,
                        int64_t ml_row, int64_t ml_slot, const Exchange ex) {
  const int row = blockIdx.x;
  const int d0 = blockIdx.y * kCombineSlice;
  pdl_launch_dependents();
  pdl_wait();
  const CombineResult c = combine_reduce(acc, m, l, NS, a_row, a_slot, ml_row, ml_slot, row, d0);
  // the counter of this (row, slice), bumped by the wait-merge kernel only
  const uint32_t step = ld_volatile_u32(ex.state + blockIdx.x * gridDim.y + blockIdx.y) + 1;
  push_to_peers(c, ex, step, D, row, d0, blockIdx.y == 0);
}

// One CTA per (row, 32-dim slice).
__global__ void __launch_bounds__(kCombineThreads)
    merge_wait_kernel(float* __restrict__ out, int D, const Exchange ex) {
  pdl_launch_dependents();
  pdl_wait();  // orders this kernel after the previous wait-merge (the step counters) and the push
  const uint32_t step = ld_volatile_u32(ex.state + blockIdx.x * gridDim.y + blockIdx.y) + 1;
  wait_merge_store(out, D, ex, step, blockIdx.x, blockIdx.y * kCombineSlice);
}

// The whole exchange in one kernel: the CTA of a (row, slice) merges this rank's split
// partials, stores the result to every rank, then waits for the same (row, slice) of every
// rank and finishes.  Pushes never wait on anything and every CTA pushes before it waits,
// so no wait can depend on a CTA that has not been scheduled: the grid (rows x D/32 CTAs of
// 256 threads) is far below one wave, and a CTA only ever waits for REMOTE stores.
__global__ void __launch_bounds__(kCombineThreads)
    combine_exchange_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                            const float* __restrict__ l, float* __restrict__ out, int NS, int D,
                            int64_t a_row, int64_t a_slot, int64_t ml_row, int64_t ml_slot,
                            const Exchange ex) {
  const int row = blockIdx.x;
  const int d0 = blockIdx.y * kCombineSlice;
  pdl_launch_dependents();
  pdl_wait();
  // bumped by the same CTA of the previous exchange
  const uint32_t step = ld_volatile_u32(ex.state + blockIdx.x * gridDim.y + blockIdx.y) + 1;
  const CombineResult c = combine_reduce(acc, m, l, NS, a_row, a_slot, ml_row, ml_slot, row, d0);
  push_to_peers(c, ex, step, D, row, d0, blockIdx.y == 0);
  wait_merge_store(out, D, ex, step, row, d0);
}

int exchange_device_status_clear() {
  const int zero = 0;
  TKV_CUDA(cudaMemcpyToSymbol(g_exchange_status, &zero, sizeof(int)));
  return TKV_OK;
}

int exchange_device_status(int* status) {
  int v = 0;
  TKV_CUDA(cudaMemcpyFromSymbol(&v, g_exchange_status, sizeof(int)));
  *status = v;
  return TKV_OK;
}

// Few partials per row (large batches: 2-8 slots): one warp per (batch, head), each
// lane a float4 slice of D, the slots walked in order.  8192 tiny CTAs of the kernel
// above would cost more in scheduling than the merge itself.
constexpr int kSmallWarps = 8;
constexpr int kSmallMaxNS = kSmallCombineMaxSlots;

template <int kMaxNS>  // compile-time bound on the slots, so no load is issued for nothing
__global__ void __launch_bounds__(kSmallWarps * 32)
    combine_small_kernel(const float* __restrict__ acc, const float* __restrict__ m,
                         const float* __restrict__ l, float* __restrict__ out,
                         float* __restrict__ out_m, float* __restrict__ out_l, int rows, int NS,
                         int D, int64_t a_row, int64_t a_slot, int64_t ml_row, int64_t ml_slot) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kSmallWarps + warp;
  if (row >= rows) return;
  pdl_wait();  // partials come from the kernel launched just before this one
  const float* mrow = m + (int64_t)row * ml_row;
  const float* lrow = l + (int64_t)row * ml_row;
  // loads first, uses afterwards: one round trip for (m, l), one for the acc rows
  float ms[kMaxNS], ls[kMaxNS];
#pragma unroll
  for (int s = 0; s < kMaxNS; ++s) {
    const int sc = min(s, NS - 1);
    ms[s] = __ldcg(mrow + sc * ml_slot);
    ls[s] = __ldcg(lrow + sc * ml_slot);
  }
  float M = -INFINITY;
#pragma unroll
  for (int s = 0; s < kMaxNS; ++s) {
    if (s >= NS) ms[s] = -INFINITY;
    M = fmaxf(M, ms[s]);
  }
  float L = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxNS; ++s) {
    ms[s] = (ms[s] > -INFINITY) ? ex2(ms[s] - M) : 0.f;  // weight of slot s
    if (ms[s] > 0.f) L = fmaf(ms[s], ls[s], L);
  }
  const float inv = (out_m == nullptr) ? (L > 0.f ? 1.f / L : 0.f) : 1.f;
  for (int v = lane; v < (D >> 2); v += 32) {
    float4 x[kMaxNS];
#pragma unroll
    for (int s = 0; s < kMaxNS; ++s) {
      const int sc = min(s, NS - 1);
      x[s] = __ldcg(reinterpret_cast<const float4*>(acc + (int64_t)row * a_row + sc * a_slot) + v);
    }
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < kMaxNS; ++s) {
      if (s < NS && ms[s] > 0.f) {  // empty slots may hold anything in acc: never use it
        a.x = fmaf(ms[s], x[s].x, a.x);
        a.y = fmaf(ms[s], x[s].y, a.y);
        a.z = fmaf(ms[s], x[s].z, a.z);
        a.w = fmaf(ms[s], x[s].w, a.w);
      }
    }
    a.x *= inv;
    a.y *= inv;
    a.z *= inv;
    a.w *= inv;
    reinterpret_cast<float4*>(out + (int64_t)row * D)[v] = a;
  }
  if (out_m != nullptr && lane == 0) {
    out_m[row] = M;
    out_l[row] = L;
  }
  // The kernel behind this one is the next step's balanced split kernel, whose CTAs must all
  // be resident at once: it may be scheduled only now, when this warp's slot is about to free.
  pdl_launch_dependents();
}

}  // namespace tkv

extern "C" int tkv_combine_strided(const float* acc, const float* m, const float* l, float* out,
                                   float* out_m, float* out_l, int64_t rows, int NS, int D,
                                   int64_t acc_row_stride, int64_t acc_slot_stride,
                                   int64_t ml_row_stride, int64_t ml_slot_stride, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(acc && m && l && out, TKV_ERR_INVALID, "combine: null pointer");
  TKV_REQUIRE((out_m == nullptr) == (out_l == nullptr), TKV_ERR_INVALID,
              "combine: out_m and out_l must be given together");
  TKV_REQUIRE(rows > 0 && NS > 0 && D > 0 && D % kCombineSlice == 0, TKV_ERR_INVALID,
              "combine: bad sizes rows=%lld NS=%d D=%d (D must be a multiple of 32)",
              (long long)rows, NS, D);
  TKV_REQUIRE(aligned16(acc) && aligned16(out) && acc_row_stride % 4 == 0 && acc_slot_stride % 4 == 0,
              TKV_ERR_ALIGN, "combine: acc and out must be 16-byte aligned, acc strides multiples of 4");
  TKV_REQUIRE(rows <= 0x7fffffffLL, TKV_ERR_INVALID, "combine: too many rows");
  if (NS <= kSmallMaxNS && rows >= kSmallCombineMinRows) {
    const unsigned blocks = (unsigned)((rows + kSmallWarps - 1) / kSmallWarps);
#define TKV_SMALL(N)                                                                          \
  TKV_CUDA(launch_pdl(tkv::combine_small_kernel<N>, dim3(blocks), dim3(kSmallWarps * 32), 0,   \
                      (cudaStream_t)stream, acc, m, l, out, out_m, out_l, (int)rows, NS, D,    \
                      acc_row_stride, acc_slot_stride, ml_row_stride, ml_slot_stride))
    if (NS <= 2) {
      TKV_SMALL(2);
    } else if (NS <= 4) {
      TKV_SMALL(4);
    } else if (NS <= 8) {
      TKV_SMALL(8);
    } else {
      TKV_SMALL(16);
    }
#undef TKV_SMALL
    return TKV_OK;
  }
  dim3 grid((unsigned)rows, D / kCombineSlice);
  TKV_CUDA(launch_pdl(tkv::combine_kernel, grid, dim3(kCombineThreads), 0, (cudaStream_t)stream, acc,
                      m, l, out, out_m, out_l, NS, D, acc_row_stride, acc_slot_stride, ml_row_stride,
                      ml_slot_stride));
  return TKV_OK;
}

extern "C" int tkv_combine(const float* acc, const float* m, const float* l, float* out,
                           float* out_m, float* out_l, int B, int HQ, int NS, int D, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(B > 0 && HQ > 0 && NS > 0 && D > 0, TKV_ERR_INVALID,
              "combine: bad sizes B=%d HQ=%d NS=%d D=%d", B, HQ, NS, D);
  return tkv_combine_strided(acc, m, l, out, out_m, out_l, (int64_t)B * HQ, NS, D,
                             (int64_t)NS * D, D, NS, 1, stream);
}

namespace {
int fill_exchange(tkv::Exchange& ex, void* const* peer_data, void* state, int world, int rank,
                  int64_t rows, int D, int wire_floats) {
  using namespace tkv;
  TKV_REQUIRE(peer_data && state, TKV_ERR_INVALID, "exchange: null pointer table");
  TKV_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, TKV_ERR_INVALID,
              "exchange: bad rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
  TKV_REQUIRE(rows > 0 && rows <= 0x7fffffffLL && D > 0 && D % kCombineSlice == 0, TKV_ERR_INVALID,
              "exchange: bad sizes rows=%lld D=%d", (long long)rows, D);
  TKV_REQUIRE((int64_t)wire_floats >= rows * (D + 2), TKV_ERR_INVALID,
              "exchange: a block of %d values cannot hold %lld rows of D=%d plus (m, l)", wire_floats,
              (long long)rows, D);
  for (int j = 0; j < world; ++j) {
    TKV_REQUIRE(peer_data[j], TKV_ERR_INVALID, "exchange: null buffer of rank %d", j);
    TKV_REQUIRE((reinterpret_cast<uintptr_t>(peer_data[j]) & 7u) == 0, TKV_ERR_ALIGN,
                "exchange: buffer of rank %d not 8-byte aligned", j);
    ex.data[j] = static_cast<uint2*>(peer_data[j]);
  }
  ex.state = static_cast<uint32_t*>(state);
  ex.world = world;
  ex.rank = rank;
  ex.rows = (int)rows;
  ex.wire = wire_floats;
  return TKV_OK;
}
}  // namespace

extern "C" int tkv_combine_push(const float* acc, const float* m, const float* l, int64_t rows, int NS,
                                int D, int64_t acc_row_stride, int64_t acc_slot_stride,
                                int64_t ml_row_stride, int64_t ml_slot_stride,
                                void* const* peer_data, void* state, int world, int rank,
                                int wire_floats, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(acc && m && l, TKV_ERR_INVALID, "combine_push: null pointer");
  TKV_REQUIRE(NS > 0, TKV_ERR_INVALID, "combine_push: NS=%d", NS);
  TKV_REQUIRE(aligned16(acc) && acc_row_stride % 4 == 0 && acc_slot_stride % 4 == 0, TKV_ERR_ALIGN,
              "combine_push: acc must be 16-byte aligned, strides multiples of 4");
  Exchange ex{};
  int rc = fill_exchange(ex, peer_data, state, world, rank, rows, D, wire_floats);
  if (rc != TKV_OK) return rc;
  dim3 grid((unsigned)rows, D / kCombineSlice);
  TKV_CUDA(launch_pdl(tkv::combine_push_kernel, grid, dim3(kCombineThreads), 0, (cudaStream_t)stream,
                      acc, m, l, NS, D, acc_row_stride, acc_slot_stride, ml_row_stride,
                      ml_slot_stride, ex));
  return TKV_OK;
}

extern "C" int tkv_combine_exchange(const float* acc, const float* m, const float* l, float* out,
                                    int64_t rows, int NS, int D, int64_t acc_row_stride,
                                    int64_t acc_slot_stride, int64_t ml_row_stride,
                                    int64_t ml_slot_stride, void* const* peer_data, void* state,
                                    int world, int rank, int wire_floats, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(acc && m && l && out, TKV_ERR_INVALID, "combine_exchange: null pointer");
  TKV_REQUIRE(NS > 0, TKV_ERR_INVALID, "combine_exchange: NS=%d", NS);
  TKV_REQUIRE(aligned16(acc) && acc_row_stride % 4 == 0 && acc_slot_stride % 4 == 0, TKV_ERR_ALIGN,
              "combine_exchange: acc must be 16-byte aligned, strides multiples of 4");
  Exchange ex{};
  int rc = fill_exchange(ex, peer_data, state, world, rank, rows, D, wire_floats);
  if (rc != TKV_OK) return rc;
  dim3 grid((unsigned)rows, D / kCombineSlice);
  TKV_CUDA(launch_pdl(tkv::combine_exchange_kernel, grid, dim3(kCombineThreads), 0,
                      (cudaStream_t)stream, acc, m, l, out, NS, D, acc_row_stride, acc_slot_stride,
                      ml_row_stride, ml_slot_stride, ex));
  return TKV_OK;
}

extern "C" int tkv_merge_wait(float* out, int64_t rows, int D, void* const* peer_data, void* state,
                              int world, int rank, int wire_floats, void* stream) {
  using namespace tkv;
  TKV_REQUIRE(out, TKV_ERR_INVALID, "merge_wait: null out");
  Exchange ex{};
  int rc = fill_exchange(ex, peer_data, state, world, rank, rows, D, wire_floats);
  if (rc != TKV_OK) return rc;
  dim3 grid((unsigned)rows, D / kCombineSlice);
  TKV_CUDA(launch_pdl(tkv::merge_wait_kernel, grid, dim3(kCombineThreads), 0, (cudaStream_t)stream, out,
                      D, ex));
  return TKV_OK;
}
