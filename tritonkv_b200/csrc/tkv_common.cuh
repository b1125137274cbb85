// Shared device/host helpers for the tritonkv_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/tritonkv_b200.h"

namespace tkv {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);

#define TKV_REQUIRE(cond, code, ...)      \
  do {                                    \
    if (!(cond)) {                        \
      ::tkv::set_error(__VA_ARGS__);      \
      return (code);                      \
    }                                     \
  } while (0)

#define TKV_CUDA(call)                                                              \
  do {                                                                              \
    cudaError_t e__ = (call);                                                       \
    if (e__ != cudaSuccess) {                                                       \
      ::tkv::set_error("%s failed: %s", #call, cudaGetErrorString(e__));            \
      return TKV_ERR_CUDA;                                                          \
    }                                                                               \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// -------------------------------------------------------------- device side
constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy; bytes past `src_bytes` are zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
// 4-, 8- or 16-byte asynchronous copy (the small sizes only exist with .ca); bytes past
// `src_bytes` are zero-filled.
template <int BYTES>
__device__ __forceinline__ void cp_async_n(uint32_t dst, const void* src, int src_bytes) {
  static_assert(BYTES == 4 || BYTES == 8 || BYTES == 16, "cp.async copies 4, 8 or 16 bytes");
  if constexpr (BYTES == 16) {
    cp_async16(dst, src, src_bytes);
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;\n" ::"r"(dst), "l"(src), "n"(BYTES),
                 "r"(src_bytes)
                 : "memory");
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}

// Shared-memory accesses by 32-bit shared address (no generic-address arithmetic).
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_v2f(uint32_t addr, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(addr), "f"(x), "f"(y) : "memory");
}

// Transpose an 8x8 matrix of 16-bit elements held one 32-bit register per lane
// (lane 4r+c holds row r, columns 2c and 2c+1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8,f32) = A * B (zero accumulator input: no register initialisation needed)
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Programmatic dependent launch: the primary kernel lets the next kernel in the stream
// start its prologue early; the dependent blocks at pdl_wait() until the primary grid has
// completed and its memory is visible.  Both are no-ops without the launch attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// Host side: launch with programmatic stream serialisation.  The kernel may begin while
// its predecessor in the stream is still running; it must call pdl_wait() before its
// first global-memory access.  After an ordinary predecessor (one that never calls
// pdl_launch_dependents) this behaves like a plain launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  __half2 h = __halves2half2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// a * b + c on f16 pairs, one rounding
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                      *reinterpret_cast<__half2*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Load element `i` of a query row of any supported dtype, rounded to f16 exactly
// as the reference's `.to(tl.float16)` does, returned as float.
__device__ __forceinline__ __half load_q_half(const void* q, int dtype, int64_t i) {
  if (dtype == TKV_DTYPE_F16) return reinterpret_cast<const __half*>(q)[i];
  if (dtype == TKV_DTYPE_BF16)
    return __float2half_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]));
  return __float2half_rn(reinterpret_cast<const float*>(q)[i]);
}

// 2^e as a float, e a compile-time-known small integer.
__host__ __device__ constexpr float pow2i(int e) {
  float r = 1.0f;
  if (e >= 0)
    for (int i = 0; i < e; ++i) r *= 2.0f;
  else
    for (int i = 0; i < -e; ++i) r *= 0.5f;
  return r;
}

}  // namespace tkv

// ------------------------------------------------- TMA / mbarrier (no cluster qualifiers)
namespace tkv {

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// Make barrier initialisation visible to the asynchronous (TMA) proxy.
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Arrival (count 1, pre-accounted in the barrier's init count) that fires when all
// cp.async copies this thread issued before it have landed.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)  // let the hardware park the warp up to ~2 us per poll
      : "memory");
  return ok;
}
// Bounded wait: gives up after `limit` polls and reports false; never spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  int limit = 1 << 22) {
  // all lanes of the warp wait on the same barrier: the vote makes the loop warp-uniform
  for (int i = 0; i < limit; ++i)
    if (__all_sync(kFullMask, mbar_try_wait(bar, parity))) return true;
  return false;
}

// 3-D tiled TMA load (c0 innermost, a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tensor_map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(dst),
      "l"(tensor_map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Warm the descriptor cache for a tensor map that lives in kernel-parameter space.
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 2-D tiled TMA load of one box into this CTA's shared memory; completion is
// signalled on `bar` as transferred bytes.  c0 = innermost coordinate (must be a
// multiple of 16 bytes), c1 = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tensor_map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(tensor_map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

}  // namespace tkv
