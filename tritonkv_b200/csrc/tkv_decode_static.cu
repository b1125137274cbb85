// Fused decode for callers that cannot hand the library any device memory of their own
// beyond inputs and output: the split partials live in a fixed device array that is part
// of the library image.
//
// Who needs this: code that runs where cudaMalloc is off limits -- inside a stream
// capture that forbids allocation, inside a serving loop whose memory pool is sized and
// frozen at start-up, or behind a host runtime that owns every byte of device memory and
// offers plugins no allocator.  Such a caller can still pass q, the packed cache and
// `out`, but has nowhere to put the (acc, m, l) partials that tkv_fused_decode wants.
#include "tkv_common.cuh"

namespace {

// 8 MiB of partials: enough for e.g. batch 64 x 32 heads x 3 slots or batch 1 x 64 heads x
// 240 slots at head_dim 128.  Every GPU that loads the library holds it until exit.
constexpr size_t kScratchFloats = size_t(2) << 20;
static __device__ __align__(256) float g_decode_scratch[kScratchFloats];

// In host code the array's name is only a handle for the runtime, not a device address,
// so the address is asked for once per device (with that device current) and cached.
// Concurrent first calls may both do the look-up and store the same value.  The cache
// does not survive cudaDeviceReset: a process that resets a device must not call this
// entry point on that device afterwards.
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};

int scratch_for_current_device(float** out) {
  int dev = 0;
  TKV_CUDA(cudaGetDevice(&dev));
  TKV_REQUIRE(dev >= 0 && dev < kMaxDevices, TKV_ERR_INVALID,
              "fused_decode_static: device index %d out of range", dev);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    TKV_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return TKV_OK;
}

}  // namespace

extern "C" int tkv_fused_decode_static(const void* q, int q_dtype, const uint8_t* k_packed,
                                       const void* k_scale, const void* k_zero,
                                       const uint8_t* v_packed, const void* v_scale,
                                       const void* v_zero, float* out, int B, int HQ, int HKV,
                                       int S, int D, int nbits, int gs, float sm_scale,
                                       void* stream) {
  using namespace tkv;
  TKV_REQUIRE(out != nullptr, TKV_ERR_INVALID, "fused_decode_static: out required");
  TKV_REQUIRE(B > 0 && HQ > 0 && HKV > 0 && S > 0 && D > 0, TKV_ERR_INVALID,
              "fused_decode_static: B, HQ, HKV, S, D must be positive");
  // one split over the whole history; the kernel balances the work across CTAs itself
  const int split_size = (S + 15) / 16 * 16;
  int nslots = 0;
  int rc = tkv_decode_plan(TKV_KERNEL_FUSED_SPLIT, nbits, D, gs, B, HQ, HKV, S, 1, split_size, 0,
                           &nslots, nullptr);
  if (rc != TKV_OK) return rc;
  // The one-time look-up of the scratch address happens on the first call on a device,
  // whatever the plan of that call, so that a warm-up call always completes the set-up.
  float* base = nullptr;
  rc = scratch_for_current_device(&base);
  if (rc != TKV_OK) return rc;
  if (nslots == 1)  // nothing to merge: the scratch is not touched
    return tkv_fused_decode(q, q_dtype, k_packed, k_scale, k_zero, v_packed, v_scale, v_zero,
                            nullptr, nullptr, nullptr, out, B, HQ, HKV, S, D, nbits, gs, sm_scale,
                            1, split_size, 1, nullptr, 0, stream);
  const size_t rows = (size_t)B * HQ * nslots;
  const size_t need = rows * ((size_t)D + 2);
  TKV_REQUIRE(need <= kScratchFloats, TKV_ERR_UNSUPPORTED,
              "fused_decode_static: B*HQ*nslots*(D+2) = %zu floats of partials exceed the built-in "
              "scratch of %zu floats (8 MiB); use tkv_fused_decode with caller-owned buffers",
              need, kScratchFloats);
  float* acc = base;
  float* m = base + rows * D;
  float* l = m + rows;
  // Every slot the combine reads is written by the split kernel in this call (data slots
  // and the m = -inf markers of unused ones), so nothing has to be cleared between calls.
  rc = tkv_fused_decode(q, q_dtype, k_packed, k_scale, k_zero, v_packed, v_scale, v_zero, acc, m, l,
                        out, B, HQ, HKV, S, D, nbits, gs, sm_scale, 1, split_size, nslots, nullptr,
                        0, stream);
  if (rc != TKV_OK) return rc;
  return tkv_combine(acc, m, l, out, nullptr, nullptr, B, HQ, nslots, D, stream);
}
