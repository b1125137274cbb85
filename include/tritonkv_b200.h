/*
 * tritonkv_b200 -- C ABI of the B200 (sm_100a) packed-KV decode-attention path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (cudaStream_t passed as void*), enqueues work on that stream, never
 * synchronises, never allocates device memory and returns an int status
 * (TKV_OK == 0).  After a non-zero status, tkv_last_error() returns a
 * thread-local, human-readable description.
 *
 * Each declaration cites the interface of the reference project (PS12007/tritonkv)
 * that it replaces, by file:line inside that project.
 *
 * Tensor layouts are the reference's, contiguous and row-major:
 *   q        (B, HQ, D)                 f16 | bf16 | f32   (rounded to f16 in-kernel)
 *   packed   (B, HKV, S, D*nbits/8)     uint8, split-P: byte j holds dims j, j+DP, ...
 *                                       in ascending nbits-wide bit slices (DP = D*nbits/8)
 *   scale,zero (B, HKV, S, D/gs)        f16, value = code*scale + zero
 *   k, v     (B, HKV, S, D)             f16 (fp16 control path)
 *   out      (B, HQ, D)                 f32
 *   acc      (B, HQ, NS, D) f32, m and l (B, HQ, NS) f32: per-split partials,
 *            acc = sum_n 2^(s_n-m) v_n, m = max_n s_n, l = sum_n 2^(s_n-m),
 *            s_n = (q.k_n)*sm_scale*log2(e)   (the exp2 domain of the reference)
 */
#ifndef TRITONKV_B200_H_
#define TRITONKV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TKV_OK 0
#define TKV_ERR_INVALID 1     /* bad argument (shape, size, null pointer)            */
#define TKV_ERR_UNSUPPORTED 2 /* valid in the reference, not built here (see text)   */
#define TKV_ERR_CUDA 3        /* a CUDA runtime call failed                          */
#define TKV_ERR_ALIGN 4       /* a base pointer is not 16-byte aligned               */

#define TKV_DTYPE_F16 0
#define TKV_DTYPE_BF16 1
#define TKV_DTYPE_F32 2

/* flags for the two decode entry points */
#define TKV_FLAG_PARTIALS_ONLY 1 /* always write (acc,m,l), even when nslots == 1 */
#define TKV_FLAG_COMBINE 2       /* with nslots > 1: enqueue tkv_combine(acc, m, l -> out) after the split kernel */
#define TKV_FLAG_K_PER_CHANNEL 4 /* tkv_fused_decode: k_scale/k_zero are (B, HKV, S/32, D), see tkv_quantize_keys_per_channel */

/* kernel ids for tkv_kernel_attrs */
#define TKV_KERNEL_FUSED_SPLIT 0
#define TKV_KERNEL_FP16_SPLIT 1
#define TKV_KERNEL_COMBINE 2
#define TKV_KERNEL_QUANTIZE_PACK 3
#define TKV_KERNEL_FUSED_SPLIT_KCHAN 4 /* the fused split kernel on per-channel keys (plans only) */

/* Library version: major*10000 + minor*100 + patch. */
int tkv_version(void);

/* Thread-local description of the last failure of any call on this thread. */
const char* tkv_last_error(void);

/* SM count, L2 size and compute capability of `device`; what the reference reads
 * from torch.cuda.get_device_properties (kernels/fused_decode_attn.py:410-413,
 * benchmark.py replicas_for :625-638). */
int tkv_device_info(int device, int* sm_count, int* l2_bytes, int* cc_major, int* cc_minor);

/* Registers / static+dynamic shared memory / local memory / resident CTAs per SM of
 * the instantiation that (nbits, D, gs) selects; replaces the Triton-cache
 * introspection of probe_gs128.py:52-77 (n_regs, n_spills, metadata.shared). */
int tkv_kernel_attrs(int kernel_id, int nbits, int D, int gs, int* regs, int* smem_bytes,
                     int* local_bytes, int* ctas_per_sm);

/* pack_codes (quantize.py:149-169): codes (rows, D) uint8 -> packed (rows, D*nbits/8). */
int tkv_pack_codes(const uint8_t* codes, uint8_t* packed, int64_t rows, int D, int nbits,
                   void* stream);

/* unpack_codes (quantize.py:172-183): the inverse. */
int tkv_unpack_codes(const uint8_t* packed, uint8_t* codes, int64_t rows, int D, int nbits,
                     void* stream);

/* quantize_groupwise (quantize.py:186-236), one launch: per-group fp32 min/max,
 * scale=(max-min)/qmax (1 if <= 0), scale and zero rounded to f16 first, then
 * code = clamp(rint((x-zero)/scale), 0, qmax), packed split-P.  Bit-exact.
 * x is (rows, D) of `in_dtype`. */
int tkv_quantize_pack(const void* x, int in_dtype, uint8_t* packed, void* scale, void* zero,
                      int64_t rows, int D, int nbits, int gs, void* stream);

/* dequantize_groupwise (quantize.py:239-246): out (rows, D) of `out_dtype`,
 * code*scale+zero evaluated in f32 then cast. */
int tkv_dequantize(const uint8_t* packed, const void* scale, const void* zero, void* out,
                   int out_dtype, int64_t rows, int D, int nbits, int gs, void* stream);

/* Work plan of a decode call: how many partial slots per (batch, query head) the split
 * kernel will write (`nslots`, the third dimension of acc/m/l) and how many CTAs it
 * launches.  kernel_id is TKV_KERNEL_FUSED_SPLIT (nbits, D, gs select the instantiation)
 * or TKV_KERNEL_FP16_SPLIT (nbits and gs ignored).  The split geometry is the
 * reference's (kernels/fused_decode_attn.py:493-499): num_splits splits of split_size
 * tokens (a multiple of 16), none empty; the kernels further cut the work into
 * equal per-CTA tile ranges, so nslots >= num_splits.  ragged != 0 plans for a call
 * that passes seq_lens. */
int tkv_decode_plan(int kernel_id, int nbits, int D, int gs, int B, int HQ, int HKV, int S,
                    int num_splits, int split_size, int ragged, int* nslots, int* grid);

/* _fused_decode_attn_split + launcher geometry (kernels/fused_decode_attn.py:155-353,
 * :493-556).  One CTA segment per (batch, KV head, history split) serves the whole GQA
 * group.  Split s covers tokens [s*split_size, min((s+1)*split_size, S_b)).  With
 * nslots == 1 (from tkv_decode_plan) and no TKV_FLAG_PARTIALS_ONLY the normalised result
 * goes to `out` and acc/m/l may be null; otherwise partials go to acc (B,HQ,nslots,D),
 * m, l (B,HQ,nslots) and `out` is untouched (call tkv_combine with NS = nslots next, or
 * pass TKV_FLAG_COMBINE to have it enqueued by the same call).
 * seq_lens (B,) int32 device pointer or null: per-sequence history length S_b <= S (no
 * reference counterpart; null == S). */
int tkv_fused_decode(const void* q, int q_dtype, const uint8_t* k_packed, const void* k_scale,
                     const void* k_zero, const uint8_t* v_packed, const void* v_scale,
                     const void* v_zero, float* acc, float* m, float* l, float* out, int B,
                     int HQ, int HKV, int S, int D, int nbits, int gs, float sm_scale,
                     int num_splits, int split_size, int nslots, const int32_t* seq_lens,
                     int flags, void* stream);

/* _fp16_decode_attn_split + launcher (kernels/fp16_decode_attn.py:47-135, :166-227):
 * the control with the identical split, scheduling, online softmax, GQA grouping and
 * partial format, K/V read as plain f16. */
int tkv_fp16_decode(const void* q, int q_dtype, const void* k, const void* v, float* acc,
                    float* m, float* l, float* out, int B, int HQ, int HKV, int S, int D,
                    float sm_scale, int num_splits, int split_size, int nslots,
                    const int32_t* seq_lens, int flags, void* stream);

/* _combine_splits (kernels/fused_decode_attn.py:355-395): log-sum-exp merge over NS
 * partials.  out (B, HQ, D).  If out_m and out_l are non-null the merged result is
 * left unnormalised in `out` with its (m, l) written there -- the wire format of a
 * cross-GPU history split; otherwise out = acc / l. */
int tkv_combine(const float* acc, const float* m, const float* l, float* out, float* out_m,
                float* out_l, int B, int HQ, int NS, int D, void* stream);

/* The same merge on partials that are not laid out (rows, NS, D): slot s of row r is at
 * acc + r*acc_row_stride + s*acc_slot_stride (floats), its m and l at
 * r*ml_row_stride + s*ml_slot_stride.  Used for the cross-GPU history split, where the
 * all-gathered buffer is (ranks, [acc | m | l]) -- no reference counterpart. */
int tkv_combine_strided(const float* acc, const float* m, const float* l, float* out, float* out_m,
                        float* out_l, int64_t rows, int NS, int D, int64_t acc_row_stride,
                        int64_t acc_slot_stride, int64_t ml_row_stride, int64_t ml_slot_stride,
                        void* stream);

/* Resident CTAs per SM x SM count for the selected split kernel: the number of
 * programs that fill the device in one wave; the launcher's target where the
 * reference uses 4 x SM count (kernels/fused_decode_attn.py:402-416). */
int tkv_wave_programs(int kernel_id, int nbits, int D, int gs, int* programs);

/* tkv_fused_decode + tkv_combine for callers that cannot provide the (acc, m, l) partial
 * buffers because they cannot allocate device memory at the point of the call: code
 * running under a frozen memory pool, inside a region where cudaMalloc is forbidden, or
 * as a plugin of a host that owns all device memory.  It has no counterpart in the
 * reference (whose launcher allocates its workspace with torch.empty).  The partials go
 * to an 8 MiB array inside the library image (held by every GPU that loads the library
 * until exit); the call itself allocates nothing.  Limit: B*HQ*nslots*(D+2) floats must
 * fit 8 MiB (nslots from tkv_decode_plan with num_splits = 1, split_size = S rounded up
 * to 16); larger problems get TKV_ERR_UNSUPPORTED.  The first call on a device looks up
 * the array's device address (one-time set-up, make it before any stream capture).  All
 * calls on a device share the array: calls that overlap on the GPU (different streams)
 * race on it -- serialise them.  Uniform history length only (no seq_lens). */
int tkv_fused_decode_static(const void* q, int q_dtype, const uint8_t* k_packed,
                            const void* k_scale, const void* k_zero, const uint8_t* v_packed,
                            const void* v_scale, const void* v_zero, float* out, int B, int HQ,
                            int HKV, int S, int D, int nbits, int gs, float sm_scale, void* stream);

/* Quantise T_new new tokens per (sequence, head) -- x (B, HKV, T_new, D) -- and write them
 * into a preallocated cache of S_cap token rows per (sequence, head): packed
 * (B, HKV, S_cap, D*nbits/8), scale / zero (B, HKV, S_cap, D/gs), at rows positions[b] + t
 * (positions int32 (B,) on the device, or null for pos0 everywhere).  Same arithmetic as
 * tkv_quantize_pack, so a cache filled token by token is byte-identical to quantising the
 * whole tensor at once.  Tokens that would fall outside [0, S_cap) are dropped.  No
 * reference counterpart: quantize.py:186-236 quantises whole tensors; this is the write
 * side of a decode loop that grows the cache one token per step. */
int tkv_quantize_append(const void* x, int in_dtype, uint8_t* packed, void* scale, void* zero, int B,
                        int HKV, int T_new, int64_t S_cap, int D, int nbits, int gs,
                        const int32_t* positions, int pos0, void* stream);

/* Keys quantised per channel: groups of 32 consecutive tokens of ONE head dimension, the
 * format the reference describes as future work (docs/future_work.md:229-293: channels that
 * are large for every token get their own scale, which makes 2-bit keys usable) and does
 * not implement -- no reference counterpart.  x (BH, S, D) keys of BH = B*HKV sequences x
 * heads; the first S_q tokens (a multiple of 32, S_q <= S) of each are quantised with the
 * per-element arithmetic of tkv_quantize_pack on the token axis: packed (BH, S_q, D*nbits/8)
 * in the same split-P byte layout, scale / zero (BH, S_q/32, D) f16.  The last S - S_q tokens
 * (a group that is not full yet) are left to the caller, who keeps them in f16.
 * tkv_fused_decode reads this format when given TKV_FLAG_K_PER_CHANNEL (values stay
 * per-token with group_size 32; S = S_q, one split, no seq_lens); the f16 tail goes through
 * tkv_fp16_decode and tkv_combine_strided merges the two partial results. */
int tkv_quantize_keys_per_channel(const void* x, int in_dtype, uint8_t* packed, void* scale, void* zero,
                                  int64_t BH, int64_t S, int64_t S_q, int D, int nbits, void* stream);

/* Cross-GPU exchange for a history split over the GPUs of one node (no reference
 * counterpart: the reference is single-GPU).  Each rank owns a receive buffer of
 * 2 * world blocks of `wire_floats` 8-byte pairs {value, step} in the layout
 * [acc rows*D | m rows | l rows], and rows * D/32 32-bit step counters (one per row and 32-dim
 * slice: `state`) in its own memory, all zeroed before the first call; the receive buffers are mapped on every rank
 * (peer or symmetric memory) and passed as a table of `world` pointers, entry j = rank j's.
 * tkv_combine_push merges this rank's split partials (arguments as tkv_combine_strided,
 * result left unnormalised) and stores them, tagged with the step number, into block
 * (step parity, rank) of every rank's buffer.  tkv_merge_wait, enqueued after it on the
 * same stream, reads the world blocks of this step -- polling each pair until it carries
 * the step -- merges them into out (rows, D) and bumps the step counters.  The wait is bounded
 * (2^18 polls, a few tenths of a second); on expiry the kernel records bit 1 of tkv_device_status and merges what
 * it has.  Ranks must call the pair in lockstep, one pair per decode step. */
int tkv_combine_push(const float* acc, const float* m, const float* l, int64_t rows, int NS, int D,
                     int64_t acc_row_stride, int64_t acc_slot_stride, int64_t ml_row_stride,
                     int64_t ml_slot_stride, void* const* peer_data, void* state, int world,
                     int rank, int wire_floats, void* stream);
int tkv_merge_wait(float* out, int64_t rows, int D, void* const* peer_data, void* state, int world,
                   int rank, int wire_floats, void* stream);

/* tkv_combine_push and tkv_merge_wait as ONE kernel (no reference counterpart): the CTA that
 * merges this rank's partials of a (row, 32-dim slice) stores the result to every rank and
 * then waits -- with the same bounded wait -- for the same slice of every rank, merges and
 * writes out (rows, D).  One kernel boundary less on the latency chain of a history-split
 * step; same buffers, step counters and lockstep rule as the pair above, with which it must
 * not be mixed within one step. */
int tkv_combine_exchange(const float* acc, const float* m, const float* l, float* out, int64_t rows,
                         int NS, int D, int64_t acc_row_stride, int64_t acc_slot_stride,
                         int64_t ml_row_stride, int64_t ml_slot_stride, void* const* peer_data,
                         void* state, int world, int rank, int wire_floats, void* stream);

/* Device-side status word of the current device (synchronises with it): 0 = ok,
 * bit 0 = a bounded wait on a copy barrier inside a decode kernel gave up (the kernel then
 * returned early and its output is invalid), bit 1 = a bounded wait for a peer's data in
 * tkv_merge_wait gave up.  No reference counterpart: the Triton kernels have no waits of
 * their own. */
int tkv_device_status(int* status);

/* Reset the status word of the current device to 0 (synchronises with it). */
int tkv_device_status_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* TRITONKV_B200_H_ */
