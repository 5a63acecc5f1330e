/* C ABI of libkf_b200: the B200 (sm_100a) implementation of KernelFuser's fused
 * Q/K RMSNorm + RoPE + GQA attention path.
 *
 * The reference has no native code; its "FFI" for this path is the pair of
 * Triton launches made by `launch_attention`
 * (src/e1_rope_publication_v1.py:661-677).  Each entry point below names the
 * reference launch it replaces.  All pointers are DEVICE pointers unless said
 * otherwise; the library never allocates or frees device memory and never
 * synchronises: every call enqueues work on the given stream and returns.
 *
 * Conventions
 *   dtype      KF_BF16 or KF_FP16; every tensor of a call shares it.
 *   layout     tensors are [B, H, S, D] with D contiguous; batch, head and
 *              row strides are given in ELEMENTS and must be positive
 *              multiples of 8 (16 bytes), base pointers 16-byte aligned.  A
 *              stride of 0 is accepted only for a dimension of size 1:
 *              expanded (broadcast) views are refused with KF_EALIGN.
 *              D is 128 or 256.
 *   tables     cos/sin are contiguous [S, D]; pass NULL for both to skip RoPE.
 *   status     device int32 owned by the caller (may be NULL only for
 *              kf_prepare_rows): stays 0 on success; a kernel whose bounded
 *              wait expired writes a positive code there (first failure wins)
 *              and returns without hanging.  The word is STICKY: while it is
 *              non-zero every attention launch that is given it returns at
 *              once without touching `out`, so that work queued behind a
 *              failure drains quickly.  The caller reads the word after
 *              synchronising and must set it back to 0 before launching
 *              again.
 *   return     0 on success; a negative KF_E* code when an argument is
 *              rejected on the host (nothing was launched);
 *              kf_last_error() then describes the reason (thread-local).
 */
#ifndef KF_B200_H_
#define KF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KF_BF16 0
#define KF_FP16 1

#define KF_OK 0
#define KF_EINVAL (-1)   /* bad shape / dtype / flag                     */
#define KF_EALIGN (-2)   /* pointer or stride not 16-byte aligned        */
#define KF_ECUDA (-3)    /* CUDA runtime / driver call failed            */
#define KF_ENOSUP (-4)   /* device is not compute capability 10.x        */

/* Library version (major*10000 + minor*100 + patch). */
int kf_version(void);

/* Message for the last non-zero return on this host thread. */
const char* kf_last_error(void);

/* Row prepare: y = RoPE(RMSNorm(x) * gamma) with position = row index s.
 * Replaces `prepare_kernel` (src/e1_rope_publication_v1.py:586-605) as launched
 * by `prepare_attention` (:652-658): called once for K (mode 'query'), and
 * also for Q in mode 'unfused'.  Rounding follows `_rows` (:551-582);
 * hf_norm = 1 rounds the normalised value before the gamma multiply,
 * hf_norm = 0 is the single-rounding 'legacy' style. */
int kf_prepare_rows(const void* x, void* y, const void* gamma, const void* cos_table, const void* sin_table,
                    int B, int H, int S, int D, int dtype, int hf_norm, float eps,
                    int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s,
                    int64_t y_stride_b, int64_t y_stride_h, int64_t y_stride_s,
                    void* stream);

/* Attention forward: out = softmax(scale * QN KN^T + mask) V with GQA head
 * mapping kv_head = q_head / (Hq / Hkv).  Replaces `attention_v2_kernel`
 * (src/e1_rope_publication_v1.py:609-649) as launched at :674-677.
 * fuse_q = 1: q is the RAW query; its RMSNorm/gamma/RoPE (gamma_q, tables,
 * eps, hf_norm) is applied in the kernel prologue (mode 'query').
 * fuse_q = 0: q is already prepared (mode 'unfused').
 * kn is the prepared K from kf_prepare_rows; v is the raw V.
 * scale is the softmax scale (the reference passes D^-0.5).
 * variant: 0 = choose automatically.  D = 128: kernel 3 when the launch has
 * at least 8192 query tiles (B*Hq*ceil(S/128)) and 2048 < S < 8192, else
 * kernel 5 (factored form: kernel 2 above 8192 tiles, else 5).  D = 256:
 * kernel 3 when the launch holds at least 200 sub-blocks of 64 keys per SM,
 * else kernel 2.
 * 1 = baseline kernel (softmax and MMA serialised inside a CTA; any head dim),
 * 2 = pipelined, warp-specialised kernel, one launch per work item (D = 128:
 * two Q tiles per CTA; D = 256: one),
 * 3 = persistent form of kernel 2: one CTA per SM takes work items from a
 * device counter and prepares the next item's Q while the running one
 * computes (D = 128 and D = 256; same results as kernel 2 bit for bit),
 * 5 = the one-tile-per-CTA kernel of D = 256 instantiated for D = 128 with
 * two CTAs per SM: faster than 2 and 3 on small problems, slower on large
 * ones.  4 is not used. */
int kf_attention_fwd(const void* q, const void* kn, const void* v, const void* gamma_q,
                     const void* cos_table, const void* sin_table, void* out,
                     int B, int Hq, int Hkv, int S, int D, int dtype,
                     int causal, int hf_norm, int fuse_q, float eps, float scale,
                     int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                     int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                     int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                     int* status, int variant, void* stream);

/* The whole operator in one call: kf_prepare_rows(k -> kn) followed by
 * kf_attention_fwd(fuse_q = 1).  Replaces `launch_attention(mode='query')`
 * (src/e1_rope_publication_v1.py:661-677), which makes the same two launches.
 * `kn` ([B, Hkv, S, D], strides n_*) is the caller's scratch for the prepared
 * K.  Same arguments and errors as the two separate calls. */
int kf_optimized_attention(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                           const void* cos_table, const void* sin_table, void* kn, void* out,
                           int B, int Hq, int Hkv, int S, int D, int dtype,
                           int causal, int hf_norm, float eps, float scale,
                           int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                           int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                           int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                           int64_t n_stride_b, int64_t n_stride_h, int64_t n_stride_s,
                           int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                           int* status, int variant, void* stream);

/* Full fusion in ONE launch, no prepared-K tensor: k is the RAW key tensor and
 * the kernel applies RMSNorm/gamma_k/RoPE to every K tile after it lands, as well
 * as the Q transform in its prologue.  Replaces `launch_attention(mode='full')`
 * (src/e1_rope_publication_v1.py:667-677; `FUSE_K`, :633-634).  The reference
 * keeps this form as an ablation (every query tile repeats the K transform) and
 * so does this library: it runs on the baseline kernel (variant 1) only.  Results
 * equal kf_prepare_rows + kf_attention_fwd(variant 1) bit for bit. */
int kf_attention_full(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                      const void* cos_table, const void* sin_table, void* out,
                      int B, int Hq, int Hkv, int S, int D, int dtype,
                      int causal, int hf_norm, float eps, float scale,
                      int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                      int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                      int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                      int* status, void* stream);

/* Factored no-RoPE form of the operator, both launches in one call.  Replaces
 * `launch_factored_attention` (src/e1_qk_publication_v3.py:638-650:
 * `prepare_factored_kernel` :593-611 + `factored_attention_kernel` :614-635).
 * kn (caller's scratch, shape of k) receives r(k * inv_rms(k) * gamma_k * gamma_q)
 * (one rounding); the RAW q feeds Q K^T and each query row's scores are scaled by
 * inv_rms(q_row) * scale * log2(e).  The reference keeps inv_rms(q) in a separate
 * FP32 tensor [B,Hq,S]; here it is computed in the attention prologue and stays on
 * chip, so there is no such argument.  No rotary tables in this form.  variant as in
 * kf_attention_fwd, restricted to 0, 2 and 5.  Opt-in: its rounding points differ from
 * kf_prepare_rows + kf_attention_fwd. */
int kf_factored_attention(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                          void* kn, void* out, int B, int Hq, int Hkv, int S, int D, int dtype, int causal,
                          float eps, float scale,
                          int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                          int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                          int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                          int64_t kn_stride_b, int64_t kn_stride_h, int64_t kn_stride_s,
                          int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                          int* status, int variant, void* stream);

/* Whole operator without any allocation (no counterpart in the reference,
 * whose wrapper always allocates its prepared-K scratch with torch.empty_like).
 * For callers that cannot allocate device memory where they call from: hosts
 * whose framework owns the device heap, code running while cudaMalloc is
 * off-limits (it synchronises the device and is illegal during stream
 * capture), request paths that must never enter the allocator.  The prepared K
 * goes to a fixed array inside the library image, so every GPU that loads the
 * library gives up kf_static_scratch_bytes() (32 MiB) until the process ends.
 *   - Runs kf_prepare_rows on k into that array, then kf_attention_fwd with
 *     fuse_q = 1; q/k/v/out/status are the caller's, as in those calls.
 *   - B*Hkv*S*D*2 bytes must fit in the array, else KF_EINVAL (nothing runs).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous
 *     call's contents.  Each call rewrites every row it later reads, so no
 *     clearing is needed, but two calls whose kernels can overlap on the GPU
 *     (different streams, no ordering) race on it: serialise them. */
size_t kf_static_scratch_bytes(void);
int kf_optimized_attention_static(const void* q, const void* k, const void* v, const void* gamma_q,
                                  const void* gamma_k, const void* cos_table, const void* sin_table, void* out,
                                  int B, int Hq, int Hkv, int S, int D, int dtype,
                                  int causal, int hf_norm, float eps, float scale,
                                  int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                  int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                  int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                                  int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                                  int* status, void* stream);

/* Self-test of the failure path (no counterpart in the reference).  Launches
 * one warp that waits, with the polling loop of the kernels' bounded waits, on
 * a barrier nobody arrives on; after `limit_clocks` SM clocks (1 .. 2^31) it
 * gives up, writes code 901 into *status and returns.  Nothing faults or
 * hangs.  Lets a host check that it notices a non-zero status word and
 * recovers from it. */
int kf_selftest_wait_timeout(int* status, long long limit_clocks, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KF_B200_H_ */
