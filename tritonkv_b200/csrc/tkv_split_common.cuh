// Pieces shared by the two split-K decode kernels (packed-KV and fp16 control):
// the launch parameters and the per-warp softmax state handed to the CTA epilogue.
#pragma once

#include "tkv_common.cuh"

namespace tkv {

constexpr int kHeadsPerCta = 8;  // query heads served per CTA (one MMA N extent)

struct DecodeParams {
  const void* q;
  int q_dtype;
  // packed cache (fused kernel)
  const uint8_t* kp;
  const uint8_t* vp;
  const __half* ks;
  const __half* kz;
  const __half* vs;
  const __half* vz;
  // fp16 cache (control kernel)
  const __half* k;
  const __half* v;
  float* acc;
  float* m;
  float* l;
  float* out;
  const int32_t* seq_lens;
  int B, HQ, HKV, S;
  int group;       // HQ / HKV
  int hchunks;     // ceil(group / 8): CTAs per KV head along the head axis
  int num_splits;
  int split_size;  // tokens per split, multiple of 16
  float qk_scale;  // sm_scale * log2(e)
  int partials;    // 1: write (acc, m, l); 0: write normalised out
  int meta_aligned;  // bytes every scale/zero tile start is aligned to: 16, 8, 4, or 0 (2 bytes only)
  int meta_phase;    // with meta_aligned == 0: the scale/zero pointers modulo 4 (0 or 2)
  int wide;          // 1: code tensors are fetched as 128-byte rows (128B TMA swizzle)
  int kv_one;        // 1: one 3-D tensor map spans the K and the V code tensor (one TMA per tile)
  int k_second;      // with kv_one: the K tensor lies above V, its tile lands second in the stage
};

// Running softmax state of one warp for the two heads (2t, 2t+1) a lane owns.
// When the warp-per-row combine kernel follows a split kernel (few partial slots, many rows):
// it lets its programmatic dependents go only at its end, which is what the balanced split
// kernel of the next step needs (see SplitLaunch::launch).
constexpr int kSmallCombineMaxSlots = 16;
constexpr int kSmallCombineMinRows = 256;

struct SoftmaxState {
  float m0, m1;  // running maxima (exp2 domain), identical across the 8 lanes sharing t
  float l0, l1;  // per-lane partial sums of p
};

}  // namespace tkv
