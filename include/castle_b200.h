/* castle_b200.h - C ABI of the B200 (sm_100a) CASTLE attention library.
 *
 * Plain pointers and sizes only.  Every device buffer, including scratch
 * ("workspace") and the status word, is allocated by the caller; unless an
 * entry point says otherwise the library allocates no device memory and keeps
 * no device state.  All launches are asynchronous on the given stream and no
 * entry point synchronises with the host.
 *
 * Return value: 0 = launched; < 0 = argument rejected (see castle_last_error());
 * > 0 = a cudaError_t raised by a launch or by tensor-map encoding.
 *
 * Device-side failures (a bounded wait that ran out) are reported through the
 * caller's `status` word: the kernels OR a non-zero code into it and return.
 *
 * Tensors are described by a base pointer and element strides over
 * (batch, head, position); the head-dim index is always contiguous.  This
 * covers both a contiguous (B,H,N,d) tensor and a view into the packed
 * projection output (B,N,6,H,d), so no copies are needed on either side.
 */
#ifndef CASTLE_B200_H
#define CASTLE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CASTLE_ABI_VERSION 1

enum { CASTLE_BF16 = 0, CASTLE_F16 = 1, CASTLE_F32 = 2 };

/* status-word bits written by kernels */
enum { CASTLE_STATUS_OK = 0, CASTLE_STATUS_WAIT_TIMEOUT = 1, CASTLE_STATUS_BAD_LAUNCH = 2 };

typedef struct {
  void* ptr;
  int64_t stride_b; /* elements between batch entries */
  int64_t stride_h; /* elements between heads */
  int64_t stride_n; /* elements between positions */
} castle_tensor_t;

typedef struct {
  int32_t batch;
  int32_t heads;
  int32_t seq_len;  /* N for the parallel pass; ignored by the decode step */
  int32_t dim_head; /* 64 or 128 for the parallel pass; 16, 32, 64 or 128 for the decode step */
  int32_t dtype;    /* CASTLE_BF16 / CASTLE_F16 (parallel pass); also CASTLE_F32 (decode step) */
  float scale;      /* multiplies qc and qu; the reference uses dim_head ** -0.5 */
} castle_problem_t;

int castle_abi_version(void);

/* Text of the last rejected call on this host thread. */
const char* castle_last_error(void);

/* ---- parallel forward ----------------------------------------------------
 * Replaces CastleAttentionFunction.forward
 * (lookahead_keys_attention/lookahead_keys_attention_triton.py:418-506, the
 * operator `castle_attention_triton(qc, kc, vc, qu, ku, vu, scale, return_U)`
 * called at lookahead_keys_attention/lookahead_keys_attention.py:122) and its
 * kernel (`_castle_attn_fwd_kernel`, same file :19-171).
 *
 * Inputs are UNSCALED, as at the reference call site.  `out` gets softmax(S)@vc,
 * `lse` (fp32, contiguous batch*heads*seq_len) the row log-sum-exp of the scores.
 * `u_out` (may be NULL; any dtype of the enum, given by `u_dtype`) gets the
 * lookahead keys U = A @ vu the cache holds; `w_state` (may be NULL; fp32,
 * contiguous batch*heads*seq_len*dim_head) gets the same matrix unrounded,
 * which castle_bwd() needs.  `workspace` holds per-tile soft-max partials.
 */
size_t castle_fwd_workspace_bytes(const castle_problem_t* p);

int castle_fwd(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
               const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
               const castle_tensor_t* vu, const castle_tensor_t* out, float* lse, const castle_tensor_t* u_out,
               int32_t u_dtype, float* w_state, void* workspace, size_t workspace_bytes, int32_t* status,
               void* stream);

/* ---- parallel forward that fills the decode caches (prefill) ---------------
 * Replaces the cache hand-off of the reference's parallel branch
 * (lookahead_keys_attention/lookahead_keys_attention.py:161-164: `U` plus the
 * unscaled qu, kc, vc become `Cache(U, qu_cache, kc_cache, vc_cache)`, which
 * the sampling loop of train_triton.py:113-139 then feeds token by token).
 * Same computation as castle_fwd(); in addition rows [0, seq_len) of the four
 * caches are written by the kernel itself: U from the final lookahead state,
 * qu/kc/vc from the tiles each key-block CTA holds in shared memory, so the
 * host needs no copy passes afterwards.  The caches are (batch, heads,
 * capacity >= seq_len, dim_head) buffers of the problem's dtype, described
 * with their own strides; rows at and beyond seq_len are left untouched.
 */
int castle_fwd_prefill(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
                       const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
                       const castle_tensor_t* vu, const castle_tensor_t* out, float* lse,
                       const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                       const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache, float* w_state,
                       void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- 16-bit element-type conversion -----------------------------------------
 * Replaces the `.half()` casts of CastleAttentionFunction
 * (lookahead_keys_attention_triton.py:437-442, :523) for bf16 callers that are
 * computed with fp16 operands: one pass over `count` contiguous elements
 * (a multiple of 8; pointers 16-byte aligned).  src_dtype CASTLE_BF16: bf16 ->
 * fp16, saturating at +-65504; CASTLE_F16: fp16 -> bf16.  `mul` (device
 * pointer to one float, may be NULL) multiplies every element on the way, which
 * is how the upstream gradient is rescaled by a power of two and the gradients
 * scaled back without a host synchronisation.
 */
int castle_convert_16bit(int32_t src_dtype, const void* src, void* dst, int64_t count, const float* mul, void* stream);

/* ---- parallel backward ---------------------------------------------------
 * Replaces CastleAttentionFunction.backward
 * (lookahead_keys_attention_triton.py:509-602) with its two kernels
 * (`_castle_attn_bwd_preprocess_do_o_dot` :175-214, `_castle_attn_bwd_kernel`
 * :218-413).  Takes the forward's inputs, `out`, `lse` and `w_state`, and the
 * upstream gradient `dout`; writes the six input gradients (same dtype as the
 * inputs; dqc and dqu already multiplied by `scale`, as at :591-592).  No
 * gradient flows through U (:512-515).  `workspace` holds fp32 accumulators
 * and, at dim_head 128, the scratch through which the pass's two kernels hand
 * three 32 KB tiles per (query block, key block) step: castle_bwd_workspace_bytes
 * asks for the accumulators plus at most 8 GiB of it, and the (batch, head)
 * pairs run in chunks of as many as fit.  A smaller workspace is accepted down
 * to the accumulators plus one pair's tiles (nblk*(nblk+1)/2 * 96 KB, nblk =
 * ceil(seq_len/128)) and only makes the chunks smaller; the error text of a
 * refused call states that least size.
 */
size_t castle_bwd_workspace_bytes(const castle_problem_t* p);

int castle_bwd(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
               const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
               const castle_tensor_t* vu, const castle_tensor_t* out, const castle_tensor_t* dout, const float* lse,
               const float* w_state, const castle_tensor_t* dqc, const castle_tensor_t* dkc,
               const castle_tensor_t* dvc, const castle_tensor_t* dqu, const castle_tensor_t* dku,
               const castle_tensor_t* dvu, void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- cached single-token step --------------------------------------------
 * Replaces the inference branch of Castle.forward
 * (lookahead_keys_attention/lookahead_keys_attention.py:166-203).
 *
 * The four caches are (batch, heads, capacity, dim_head) buffers holding
 * `cache_len` valid rows.  The step rewrites U[0..cache_len) in place
 * (U[k] += sigmoid(scale * qu_cache[k] . ku) * vu, :182-183), appends row
 * `cache_len` to all four (a zero row for U, :185-188,202) and writes the
 * attention output for the new token (:190-200).  Requires cache_len < capacity.
 * The six `*_new` tensors are the new token's (batch, heads, 1, dim_head) rows,
 * unscaled.  `workspace` holds split partials.  Caches whose position stride equals dim_head (rows adjacent in
 * memory, at least 128 bytes each) take the fastest path.
 */
size_t castle_decode_workspace_bytes(const castle_problem_t* p, int32_t cache_len);

int castle_decode_step(const castle_problem_t* p, int32_t cache_len, int32_t capacity,
                       const castle_tensor_t* qc_new, const castle_tensor_t* kc_new, const castle_tensor_t* vc_new,
                       const castle_tensor_t* qu_new, const castle_tensor_t* ku_new, const castle_tensor_t* vu_new,
                       const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                       const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache, const castle_tensor_t* out,
                       void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ---- cached single-token step without caller scratch -----------------------
 * (no counterpart in the reference)  Same step and same arguments as
 * castle_decode_step(), minus the workspace: the split partials go to a fixed
 * 520 KiB array built into the library, which every GPU that loads the library
 * holds until the process exits.  Meant for hosts that cannot allocate device
 * memory on the token path (an engine whose own arena already owns the device,
 * or a non-torch host that binds only this ABI).  It calls no allocator of any
 * kind.  Limit: batch * heads * row-splits <= 1024 and dim_head <= 128; larger
 * problems are rejected (< 0) with a message naming the limit - use
 * castle_decode_step() for those.  The first call on each device looks up the
 * array's device address (cudaGetSymbolAddress, with that device current); make
 * that first call before starting any stream capture.  All calls on a device
 * share the one array, so two calls whose kernels overlap on the GPU (different
 * streams, or different host threads) race; calls on one stream are safe.
 */
int castle_decode_step_static(const castle_problem_t* p, int32_t cache_len, int32_t capacity,
                              const castle_tensor_t* qc_new, const castle_tensor_t* kc_new,
                              const castle_tensor_t* vc_new, const castle_tensor_t* qu_new,
                              const castle_tensor_t* ku_new, const castle_tensor_t* vu_new,
                              const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                              const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache,
                              const castle_tensor_t* out, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CASTLE_B200_H */
