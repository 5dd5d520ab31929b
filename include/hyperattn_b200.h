/*
 * C ABI of libhyperattn_b200.so -- the B200 (sm_100a) kernels behind the HyperAttention module.
 *
 * Every entry point takes raw device pointers, element counts/strides and a CUDA stream (as void*), returns an
 * int status (HA_OK or a negative HA_ERR_* for rejected arguments, a positive value for a condition reported by
 * the device through a status word) and never allocates or frees device memory: outputs and workspaces are the
 * caller's.  Nothing here synchronises the stream.
 *
 * Each declaration cites the interface of the reference project (amirzandieh/HyperAttention, paths relative to
 * its root) that it stands in for.
 */
#ifndef HYPERATTN_B200_H
#define HYPERATTN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  HA_OK = 0,
  HA_ERR_INVALID = -1,      /* a shape/stride/size the kernels do not accept (reference: AssertionError) */
  HA_ERR_DTYPE = -2,        /* unsupported element type */
  HA_ERR_WORKSPACE = -3,    /* workspace pointer null or too small */
  HA_ERR_CUDA = -4,         /* a CUDA runtime call (launch, attribute) failed; see ha_last_cuda_error */
  HA_ERR_TOO_LARGE = -5,    /* beyond a size limit of the entry point: a grid dimension (segments, work items), or the
                               built-in scratch array of ha_seg_sort_noalloc */
  HA_DEV_TIMEOUT = 1,       /* a bounded device-side wait gave up (written to the caller's status word) */
  HA_DEV_BAD_INDEX = 2,     /* HA_FLAG_CHECK_INDICES: q_idx / k_idx / sample_idx holds a row outside its segment */
  HA_DEV_BAD_LAUNCH = 3     /* a kernel found its shared-memory window smaller than its layout needs and did no work */
};

enum { HA_BF16 = 0, HA_FP16 = 1, HA_FP32 = 2 };

/* attention patterns */
enum {
  HA_MODE_HYPER = 0,        /* sorted block-diagonal windows + sampled rows */
  HA_MODE_FLASH = 1         /* exact attention over contiguous rows, optional causal mask */
};

/* flags */
enum {
  HA_FLAG_CAUSAL = 1,        /* HA_MODE_FLASH: key j visible to query i iff j <= i */
  HA_FLAG_SMOOTH = 2,        /* HA_MODE_HYPER: windows centred on the 128-row tile (smooth_block=True) */
  HA_FLAG_MERGE = 4,         /* forward: combine with the (o, lse) already in the output buffers */
  HA_FLAG_MERGE_EXACT = 8,   /* with MERGE: plain log-sum-exp combine instead of the reference's rounded formula */
  HA_FLAG_BWD_REF_SMOOTH = 16,/* backward + SMOOTH: enumerate pairs per key tile as the reference backward does */
  HA_FLAG_FORCE_SIMT = 32,   /* use the fp32 CUDA-core kernels even where a tensor-core kernel exists */
  HA_FLAG_NO_WS = 128,       /* keep the earlier kernels (forward: one tile per CTA; backward: one thread-block role) where the
                                persistent warp-specialised ones apply */
  HA_FLAG_CHECK_INDICES = 256,/* HA_MODE_HYPER, needs `status`: a checking kernel runs first and looks at every entry of q_idx, k_idx
                                and sample_idx; an entry outside [0, rows of the segment) sets the status words to
                                HA_DEV_BAD_INDEX, and the attention kernel that follows returns at once instead of reading
                                (and faulting on) a row that does not exist.  The reference relies on its caller here
                                (torch.sort cannot produce such an index; a hand-made permutation can). */
  HA_FLAG_BWD_KV_INIT = 64   /* backward, HA_MODE_FLASH with m_q <= 2048 on the tensor-core kernel: dk_acc / dv_acc hold
                                garbage; the launch stores (not adds) every key row of every segment */
};

const char* ha_version(void);
const char* ha_last_cuda_error(void);

/* --------------------------------------------------------------------------------------------------------------
 * Angular LSH.  Replaces AngularLSHTriton.hash_triton / _angular_lsh / _angular_lsh_kernel
 * (src/angular_lsh_triton.py:181-182, :99-145, :14-96):
 *   codes[b,h,i] = gray( sum_j 2^j [ x[b,h,i,:] . proj[:,j] > 0 ] ),  gray(c) = c ^ (c >> 1).
 * x: [B,H,n,d] with element strides (last dim contiguous), dtype HA_*; proj: d*r floats, row-major [d][r], the
 * module's proj_dir converted to float; codes: int32 [B,H,n] contiguous.  1 <= r <= 16, d <= 256.
 */
int ha_lsh_hash(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_n, int32_t B, int32_t H, int32_t n,
                int32_t d, int32_t dtype, const float* proj, int32_t r, int32_t* codes, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Segmented stable argsort of bucket codes.  Replaces torch.sort(codes, dim=2, stable=True)[1]
 * (hyper_attention.py:116-117), for all segments of one call at once.
 * codes: int32 [rows][n].  Each row is cut into n/span spans; in every span the seg_len keys starting at seg_off
 * form one segment.  idx_out: int32 [rows * (n/span)][seg_len], positions local to the segment (0..seg_len-1),
 * ascending by code, ties in original order.  key_bits = number of significant code bits (<= 16).
 * (rows = B*H, span = n, seg_off = 0, seg_len = n is the plain per-head sort.)
 */
int64_t ha_seg_sort_workspace_bytes(int32_t rows, int32_t n, int32_t span, int32_t seg_len, int32_t key_bits);
int ha_seg_sort(const int32_t* codes, int32_t rows, int32_t n, int32_t span, int32_t seg_off, int32_t seg_len,
                int32_t key_bits, int32_t* idx_out, void* workspace, int64_t workspace_bytes, void* stream);

/* The same sort for callers that have no memory to give: embedders that cannot call cudaMalloc themselves (all of
 * device memory already belongs to their own pools, or they sit in a region where an allocation -- and the device-wide
 * synchronisation it implies -- is not allowed) and do not link an allocator such as torch's.  The scratch is a fixed
 * array of HA_SEG_SORT_STATIC_BYTES inside the library image, resident on every GPU that loads the library until the
 * process exits.  This entry point has no counterpart in the reference; it exists only for such embedders.
 *   - Inputs and the output are still the caller's.  No cudaMalloc, cudaFree or other allocating routine is called.
 *   - A sort that would need more than HA_SEG_SORT_STATIC_BYTES of scratch (ha_seg_sort_workspace_bytes tells) is
 *     refused with HA_ERR_TOO_LARGE and nothing is launched.  With 8-bit keys that is 4096 sub-chunks of 1024 keys,
 *     e.g. 32 heads x 131072 tokens.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array and find in it whatever the previous call left; nothing in it needs
 *     clearing, because each call writes every word before reading it.  Two calls that overlap on the GPU (different
 *     streams, or different host threads) race on it: serialise them.
 */
#define HA_SEG_SORT_STATIC_BYTES (4u << 20)
int ha_seg_sort_noalloc(const int32_t* codes, int32_t rows, int32_t n, int32_t span, int32_t seg_off, int32_t seg_len,
                        int32_t key_bits, int32_t* idx_out, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Row gather: dst[g, i, :] = src[head(g), base(g) + idx[g, i], :].  Replaces indexing()
 * (src/attn_utils.py:27-50; x.gather(2, idx.expand(...))).  width = row length in elements.
 */
int ha_gather_rows(const void* src, int64_t stride_b, int64_t stride_h, int64_t stride_n, int32_t B, int32_t H,
                   int32_t width, int32_t dtype, const int32_t* idx, int32_t n_idx, void* dst, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Attention forward and backward over "segments".
 *
 * Tensors are [B,H,n,*] with element strides; a call works on segs_per_head segments per (b,h): segment p of head
 * (b,h) has its queries at rows p*span + q_off + [0, m_q) and its keys/values at rows p*span + k_off + [0, m_k).
 * The plain call has segs_per_head = 1, span = n, offsets 0.  The causal recursion's rectangle at depth l has
 * segs_per_head = 2^l, span = n/2^l, q_off = span/2, k_off = 0, m_q = m_k = span/2; its leaves have span = m_q = m_k.
 *
 * HA_MODE_HYPER replaces hyper_attn_func / _fwd_hyper_kernel (src/hyper_attn_triton.py:895-948, :26-192) and, in
 * the backward, _bwd_preprocess_do_o_dot, _bwd_permuted_block_diagonal_kernel and _bwd_sampled_col_kernel
 * (:196-236, :399-506, :517-665).  q_idx / k_idx: int32 [B*H*segs_per_head][m] local sorted positions -> local row;
 * sample_idx: int32 [B*H*segs_per_head][sample_size] local key rows (NULL = 0..sample_size-1, the reference's choice).
 * sample_logw / sample_mask (both or neither; outputs of ha_sample_weights): the sampled rows become an importance-
 * weighted estimate of the keys outside each query tile's block window.  No counterpart in the reference's code,
 * whose sampled part always reads rows 0..sample_size-1 unweighted (src/hyper_attn_triton.py:139-176).
 * HA_MODE_FLASH replaces flash_attn_func / _fwd_kernel / _bwd_kernel (src/flash_attn_triton.py:995-1042, :57-267,
 * :651-792) without the bias branch.
 *
 * With HA_FLAG_MERGE the forward combines its result with the (o, lse) already stored for the same rows, as
 * add_self_attentions does (src/attn_utils.py:6-24) with the stored values as attn1/lse1.  If part_o/part_lse are
 * given, the un-merged result of this call is also written there ([B,H,n,dv] layout of o / [B,H,n] of lse).
 */
typedef struct {
  int32_t mode, flags, dtype;
  int32_t B, H, n;                 /* tensor extents; n = rows per head in q, k, v, o */
  int32_t d, dv;
  int32_t segs_per_head, span, q_off, k_off, m_q, m_k;
  int32_t block_size, sample_size; /* HA_MODE_HYPER */
  int32_t kv_group;                /* grouped-query attention: this many consecutive query heads share one K/V head (0 or 1:
                                      none).  k, v, k_idx, sample_idx and the dK/dV accumulators then have H / kv_group heads
                                      (K is hashed and sorted once per group, never expanded -- the reference can only be
                                      given expanded heads, chatglm_fast_attention.py:53-58); the backward sums a group's
                                      contributions in the fp32 accumulators (no direct dK/dV outputs) */
  float scale;
  const void *q, *k, *v;
  int64_t q_sb, q_sh, q_sn, k_sb, k_sh, k_sn, v_sb, v_sh, v_sn;
  const int32_t *q_idx, *k_idx, *sample_idx;
  /* forward outputs (backward: inputs) */
  void* o;
  int64_t o_sb, o_sh, o_sn;
  float* lse;                      /* [B,H,n] contiguous */
  void* part_o;                    /* optional, same strides as o */
  float* part_lse;                 /* optional */
  /* backward only */
  const void* d_o;                 /* gradient of o, strides do_s* */
  int64_t do_sb, do_sh, do_sn;
  const float* delta;              /* [B,H,n]: sum_d o*do of the part this call differentiates */
  float *dq_acc, *dk_acc, *dv_acc; /* fp32 [B,H,n,d], [B,H,n,d], [B,H,n,dv] contiguous accumulators (added into) */
  int32_t* status;                 /* optional device status word (0 = ok) */
  int32_t* status_host;            /* optional word in pinned (device-visible) host memory that gets the same value: the
                                      host can look at it between calls without synchronising the stream */
  const float* sample_logw;        /* optional [B*H*segs_per_head][m_q/128]: log weight of the kept sampled slots */
  const uint32_t* sample_mask;     /* optional [B*H*segs_per_head][m_q/128][sample_size/32]: bit s = slot s dropped */
  /* backward, HA_MODE_HYPER on the tensor-core kernel only (ha_attn_bwd_uses_tensor_cores): direct dK/dV.  Every key
   * row's block part is complete inside one work item, so it is stored straight into dk_out / dv_out (dtype rows,
   * [B,H,n,d] / [B,H,n,dv] contiguous, every row of every segment written); the sampled rows' extra terms are summed in
   * the small slot-indexed fp32 buffers dk_sacc / dv_sacc (B*H*segs_per_head * sample_size * d / ... * dv floats, zeroed
   * by the caller; the order of the floats inside is the library's own) and added by ha_attn_bwd_finish, which must get
   * the same parameters.  dk_acc / dv_acc are not used then.  sample_idx rows must be distinct.
   * Same arithmetic as the reference, whose sampled-column kernel adds onto the dk / dv its block kernel stored
   * (src/hyper_attn_triton.py:399-506, :517-665). */
  void *dk_out, *dv_out;
  float *dk_sacc, *dv_sacc;
  /* direct dQ (only where ha_attn_bwd_direct_level says 2; together with dk_out / dv_out): every query tile's dQ is summed
   * inside one work item (a 256-row block's two key tiles and the two sampled key tiles against its two query tiles) and
   * written once to dq_out ([B,H,n,d] contiguous, dtype rows): no fp32 accumulator, zero-fill or cast pass; dq_acc is
   * not used and may be NULL. */
  void* dq_out;
} ha_attn_params;

int ha_attn_fwd(const ha_attn_params* p, void* stream);
int ha_attn_bwd(const ha_attn_params* p, void* stream);
/* Which direct outputs ha_attn_bwd accepts for these parameters (dtype, head dims, flags, sizes, strides and pointer
 * alignment are looked at): 0 = none (fp32 accumulators only), 1 = dk_out / dv_out, 2 = dq_out as well (head dims 64,
 * block size 129..256 on whole blocks, plain windows, 0 or 256 sampled rows). */
int ha_attn_bwd_direct_level(const ha_attn_params* p);
/* After ha_attn_bwd with dk_out / dv_out: dk_out[row of slot s] += dk_sacc[s] (same for dv), in the tensors' dtype. */
int ha_attn_bwd_finish(const ha_attn_params* p, void* stream);

/* Weights of uniformly sampled key columns (no counterpart in the reference's code; its paper's estimator).
 * For every sorted query tile t of every segment: slot s of sample_idx is dropped (mask bit set) when that key's
 * sorted position lies inside the tile's block window, and tile_logw = log((m - window size) / kept slots), so that
 * the kept samples stand for all keys outside the window (-inf when none is kept).  m = rows per segment (a
 * multiple of 128), sample_size a multiple of 128; sample_idx entries must be distinct rows in [0, m).
 * inv_workspace: int32 [segs][m] scratch.  tile_logw: [segs][m/128].  tile_mask: [segs][m/128][sample_size/32]. */
int ha_sample_weights(const int32_t* k_idx, const int32_t* sample_idx, int32_t segs, int32_t m, int32_t block_size,
                      int32_t sample_size, int32_t smooth, int32_t* inv_workspace, float* tile_logw,
                      uint32_t* tile_mask, void* stream);

/* delta[b,h,i] = sum_e o[b,h,i,e] * do[b,h,i,e].  Replaces _bwd_preprocess_do_o_dot (src/hyper_attn_triton.py:196-236,
 * src/flash_attn_triton.py:271-312). */
int ha_delta(const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn, const void* d_o, int64_t do_sb, int64_t do_sh,
             int64_t do_sn, int32_t B, int32_t H, int32_t n, int32_t dv, int32_t dtype, float* delta, void* stream);

/* dst (dtype) = src (fp32), contiguous count elements.  Replaces dq.copy_(dq_accum) (src/hyper_attn_triton.py:892). */
int ha_cast_from_f32(const float* src, void* dst, int64_t count, int32_t dtype, void* stream);

/* Stand-alone merge.  Replaces add_self_attentions (src/attn_utils.py:6-24) on [rows, dv] / [rows] contiguous data:
 * (o1, lse1) <- merge((o1, lse1), (o2, lse2)); exact != 0 selects the un-rounded log-sum-exp form. */
int ha_lse_merge(void* o1, float* lse1, const void* o2, const float* lse2, int64_t rows, int32_t dv, int32_t dtype,
                 int32_t exact, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Causal HyperAttention in one call.  Replaces the recursion in HyperAttention.forward (hyper_attention.py:51-96)
 * for the regular case (n divisible by 2^levels, every rectangle a multiple of 128 rows): hashes q and k once,
 * sorts the segments of every depth, runs the exact leaves and the rectangles deepest first, merging in place.
 * levels = number of half-splits (n / 2^levels <= min_seq_len < n / 2^(levels-1)).
 * min_seq_len: the module's threshold.  The deepest rectangles have n / 2^levels rows a side; where that is below
 * min_seq_len the reference computes them exactly (forward_no_causal_mask, hyper_attention.py:109-113), and so does
 * this call (HA_MODE_FLASH without mask, merged like the others).  0 = every rectangle takes the hyper pattern.
 * saved: workspace that the matching backward call needs again (sort indices of every depth, per-part outputs
 * when keep_parts != 0); scratch: workspace free after the call returns.
 */
typedef struct {
  int32_t dtype, flags;            /* flags: HA_FLAG_SMOOTH, HA_FLAG_MERGE_EXACT, HA_FLAG_BWD_REF_SMOOTH, HA_FLAG_FORCE_SIMT, HA_FLAG_NO_WS */
  int32_t B, H, n, d, dv;
  int32_t levels, block_size, sample_size, lsh_bits, keep_parts;
  int32_t min_seq_len;
  int32_t kv_group;                /* as in ha_attn_params: k, v (and dk, dv_out) are [B, H / kv_group, n, *] */
  float scale;
  const void *q, *k, *v;           /* [B,H,n,*] contiguous */
  const float* proj;               /* [d][lsh_bits] */
  void* o;                         /* [B,H,n,dv] contiguous */
  float* lse;                      /* [B,H,n] */
  void* saved;  int64_t saved_bytes;
  void* scratch; int64_t scratch_bytes;
  /* backward only */
  const void* d_o;                 /* [B,H,n,dv] contiguous */
  void *dq, *dk, *dv_out;          /* [B,H,n,*] contiguous, dtype */
  int32_t* status;
  int32_t* status_host;            /* as in ha_attn_params */
} ha_causal_params;

int64_t ha_causal_saved_bytes(const ha_causal_params* p);
/* Scratch of one call (contents undefined afterwards).  The forward's includes room for every part's (o, lse) when the call
 * keeps no parts for a backward and they fit 16 GB: the merges then run as one pass over the parts instead of in every
 * rectangle's epilogue. */
int64_t ha_causal_scratch_bytes(const ha_causal_params* p, int32_t backward);
int ha_causal_fwd(const ha_causal_params* p, void* stream);
int ha_causal_bwd(const ha_causal_params* p, void* stream);

/* The non-causal module call in one call each way.  Replaces forward_no_causal_mask on sequences of at least
 * min_seq_len (hyper_attention.py:103-132: hash, stable sort, hyper_attn_func) and its backward (delta, the backward kernel
 * with the direct outputs it supports, the finishing pass), on contiguous [B,H,n,*] tensors, sampled rows 0..sample_size-1.
 * Takes the same parameter struct as the causal schedule; levels, keep_parts and min_seq_len are not looked at.  saved holds the two sort permutations
 * (needed again by the backward); scratch is free after each call. */
int64_t ha_noncausal_saved_bytes(const ha_causal_params* p);
int64_t ha_noncausal_scratch_bytes(const ha_causal_params* p, int32_t backward);
int ha_noncausal_fwd(const ha_causal_params* p, void* stream);
int ha_noncausal_bwd(const ha_causal_params* p, void* stream);

/* Diagnostic for the timeout path.  One warp polls an mbarrier that nothing ever arrives at, `polls` times (1..2^18),
 * gives up and reports HA_DEV_TIMEOUT through status / status_host exactly as the attention kernels do when one of their
 * bounded waits runs out.  No copy and no tensor-core operation is in flight; the kernel returns normally and the
 * context stays usable.  No counterpart in the reference (its Triton kernels have no waits to bound). */
int ha_wait_probe(int32_t* status, int32_t* status_host, int32_t polls, void* stream);

/* Number of kernels this library has launched in the calling process (all entry points, all streams). */
int64_t ha_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
