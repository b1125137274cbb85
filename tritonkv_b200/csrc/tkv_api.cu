// Library-level entry points: error text, device facts, kernel resource queries.
#include <stdarg.h>

#include "tkv_splitk_driver.cuh"

namespace tkv {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fused_attrs(int nbits, int D, int gs, int* regs, int* smem, int* local, int* ctas);
int fp16_attrs(int D, int* regs, int* smem, int* local, int* ctas);
int fused_device_status(int* status);
int fp16_device_status(int* status);
int exchange_device_status(int* status);
int fused_device_status_clear();
int fp16_device_status_clear();
int exchange_device_status_clear();
int fused_plan(int nbits, int D, int gs, SplitSched* sc, int B, int HKV, int hchunks, int S,
               int num_splits, int split_size, bool ragged, bool kchan);
int fp16_plan(int D, SplitSched* sc, int B, int HKV, int hchunks, int S, int num_splits,
              int split_size, bool ragged);

}  // namespace tkv

using namespace tkv;

extern "C" int tkv_version(void) { return 100; }

extern "C" const char* tkv_last_error(void) { return g_error; }

extern "C" int tkv_device_info(int device, int* sm_count, int* l2_bytes, int* cc_major,
                               int* cc_minor) {
  int v = 0;
  if (sm_count) {
    TKV_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
    *sm_count = v;
  }
  if (l2_bytes) {
    TKV_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, device));
    *l2_bytes = v;
  }
  if (cc_major) {
    TKV_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, device));
    *cc_major = v;
  }
  if (cc_minor) {
    TKV_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, device));
    *cc_minor = v;
  }
  return TKV_OK;
}

extern "C" int tkv_kernel_attrs(int kernel_id, int nbits, int D, int gs, int* regs,
                                int* smem_bytes, int* local_bytes, int* ctas_per_sm) {
  switch (kernel_id) {
    case TKV_KERNEL_FUSED_SPLIT:
      return fused_attrs(nbits, D, gs, regs, smem_bytes, local_bytes, ctas_per_sm);
    case TKV_KERNEL_FP16_SPLIT:
      return fp16_attrs(D, regs, smem_bytes, local_bytes, ctas_per_sm);
  }
  set_error("kernel_attrs: kernel id %d has no per-instantiation attributes", kernel_id);
  return TKV_ERR_INVALID;
}

extern "C" int tkv_decode_plan(int kernel_id, int nbits, int D, int gs, int B, int HQ, int HKV,
                               int S, int num_splits, int split_size, int ragged, int* nslots,
                               int* grid) {
  TKV_REQUIRE(B > 0 && HQ > 0 && HKV > 0 && S > 0 && HQ % HKV == 0, TKV_ERR_INVALID,
              "decode_plan: bad sizes B=%d HQ=%d HKV=%d S=%d", B, HQ, HKV, S);
  TKV_REQUIRE(num_splits >= 1 && split_size >= 16 && split_size % 16 == 0 &&
                  (int64_t)num_splits * split_size >= S && (int64_t)(num_splits - 1) * split_size < S,
              TKV_ERR_INVALID, "decode_plan: %d splits of %d tokens must cover S=%d with no empty split",
              num_splits, split_size, S);
  const int hchunks = (HQ / HKV + kHeadsPerCta - 1) / kHeadsPerCta;
  SplitSched sc;
  int rc;
  if (kernel_id == TKV_KERNEL_FUSED_SPLIT || kernel_id == TKV_KERNEL_FUSED_SPLIT_KCHAN)
    rc = fused_plan(nbits, D, gs, &sc, B, HKV, hchunks, S, num_splits, split_size, ragged != 0,
                    kernel_id == TKV_KERNEL_FUSED_SPLIT_KCHAN);
  else if (kernel_id == TKV_KERNEL_FP16_SPLIT)
    rc = fp16_plan(D, &sc, B, HKV, hchunks, S, num_splits, split_size, ragged != 0);
  else {
    set_error("decode_plan: kernel id %d is not a split kernel", kernel_id);
    return TKV_ERR_INVALID;
  }
  if (rc != TKV_OK) return rc;
  if (nslots) *nslots = sc.nslots;
  if (grid) *grid = sc.grid;
  return TKV_OK;
}

extern "C" int tkv_wave_programs(int kernel_id, int nbits, int D, int gs, int* programs) {
  TKV_REQUIRE(programs, TKV_ERR_INVALID, "wave_programs: null output");
  int ctas = 0, sms = 0, dev = 0;
  int rc = tkv_kernel_attrs(kernel_id, nbits, D, gs, nullptr, nullptr, nullptr, &ctas);
  if (rc != TKV_OK) return rc;
  TKV_CUDA(cudaGetDevice(&dev));
  TKV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  *programs = ctas * sms;
  return TKV_OK;
}

extern "C" int tkv_device_status(int* status) {
  TKV_REQUIRE(status, TKV_ERR_INVALID, "device_status: null output");
  int a = 0, b = 0, c = 0;
  int rc = fused_device_status(&a);
  if (rc != TKV_OK) return rc;
  rc = fp16_device_status(&b);
  if (rc != TKV_OK) return rc;
  rc = exchange_device_status(&c);
  if (rc != TKV_OK) return rc;
  *status = a | b | (c << 1);
  return TKV_OK;
}

extern "C" int tkv_device_status_clear(void) {
  int rc = fused_device_status_clear();
  if (rc != TKV_OK) return rc;
  rc = fp16_device_status_clear();
  if (rc != TKV_OK) return rc;
  return exchange_device_status_clear();
}
