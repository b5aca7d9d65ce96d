/*
 * come_b200 -- C ABI of the B200 (sm_100a) kernels for the Co-Me accelerated-inference hot path:
 * confidence-guided window selection, token merge into a packed variable-length sequence, biased
 * variable-length attention, and unmerge.
 *
 * Conventions
 *   - every pointer named *_dev is DEVICE memory on the current CUDA device; nothing here allocates or
 *     frees device memory, the caller owns every buffer (outputs and workspaces included);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and nothing synchronises;
 *   - functions return COME_OK (0) or a negative COME_ERR_* code and never throw; a human-readable
 *     message for the last failure on the calling thread is available from come_last_error();
 *   - dtype is COME_F32 / COME_F16 / COME_BF16.
 *
 * Each entry point names the interface of the reference project (paths relative to its root) it replaces.
 */
#ifndef COME_B200_H
#define COME_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COME_B200_VERSION 100

enum { COME_F32 = 0, COME_F16 = 1, COME_BF16 = 2 };

enum {
    COME_OK = 0,
    COME_ERR_ARG = -1,         /* invalid argument (shape, alignment, null pointer) */
    COME_ERR_CUDA = -2,        /* a CUDA runtime / driver call failed */
    COME_ERR_UNSUPPORTED = -3, /* valid request that this build deliberately does not implement */
    COME_ERR_DEVICE = -4       /* a kernel raised the device status word (bounded wait ran out) */
};

/* selection modes / scopes of come_select_windows */
enum { COME_SELECT_RANK = 0, COME_SELECT_ABS = 1, COME_SELECT_ZSCORE = 2 };
enum { COME_SCOPE_BATCH = 0, COME_SCOPE_FRAME = 1 };

/*
 * Token order of one frame.  grid_h == 0 selects the 1-D operator: `n_groups` groups of `group_w`
 * consecutive tokens behind `start_index` special tokens (N = start_index + n_groups * group_w).
 * grid_h > 0 selects the 2-D operator on a row-major grid_h x grid_w patch grid behind the special tokens
 * (N = start_index + grid_h * grid_w): group_h x group_w windows tile the top-left
 * floor(grid_h/group_h)*group_h x floor(grid_w/group_w)*group_w region in raster order; patches outside
 * that region are never merged and are emitted, in row-major order, directly after the special tokens.
 */
typedef struct come_layout {
    int32_t start_index;
    int32_t grid_h, grid_w;
    int32_t group_h, group_w;
    int32_t n_groups; /* 1-D only; ignored (derived) for the 2-D operator */
} come_layout_t;

int come_version(void);
const char *come_last_error(void);

/* Number of groups (windows) per frame, tokens per frame and never-merged prefix length of a layout. */
int come_layout_info(const come_layout_t *layout, int64_t *n_groups, int64_t *tokens_per_frame,
                     int64_t *prefix_len);

/*
 * Window selection: per-patch confidence -> boolean merge mask.
 * Replaces the tensor code of _CoMe_2D_Base.build_ctx (src/accelerate/token_merger/co_me_2d.py:268-298)
 * and CoMe_TokenMerger.build_ctx (src/accelerate/token_merger/co_me.py:54-73).
 *   conf_dev   [batch, frames_per_batch * grid_h * grid_w], dtype
 *   mask_dev   [batch * frames_per_batch, M] uint8 (0/1), M = floor(grid_h/group_h) * floor(grid_w/group_w)
 *   mode       COME_SELECT_RANK: mask = mean < quantile(mean, threshold) (linear interpolation, float32);
 *              COME_SELECT_ABS : mask = mean < threshold
 *              COME_SELECT_ZSCORE: the confidences of a batch element are first normalised, (x - mean) / (std + 1e-3)
 *                                with the unbiased standard deviation over all its frames (co_me_2d.py:274-281,
 *                                co_me.py:54-59), then mask = mean of the normalised window < threshold; scope is ignored
 *              In the last two modes the threshold is rounded to dtype before the comparison, as PyTorch does when a
 *              tensor is compared with a Python number.
 *   scope      COME_SCOPE_BATCH: one quantile per batch element over all its frames (2-D merger class);
 *              COME_SCOPE_FRAME: one quantile per frame (1-D merger class, standalone op chain)
 * At most 32768 windows per quantile group.
 * A NaN confidence: the reference's quantile of a group that holds a NaN is NaN and nothing of that group is merged; here
 * the sort leaves a NaN where it stands and the threshold is unspecified.  Callers must pass finite confidences.
 */
int come_select_windows(const void *conf_dev, int dtype, int64_t batch, int64_t frames_per_batch, int grid_h,
                        int grid_w, int group_h, int group_w, float threshold, int mode, int scope,
                        uint8_t *mask_dev, void *stream);

/*
 * Ranking selection with one quantile level per quantile group instead of one for all: ratios_dev holds one float in
 * [0, 1] (values outside are clamped) per batch element (COME_SCOPE_BATCH) or per frame (COME_SCOPE_FRAME).  Same
 * arithmetic as come_select_windows otherwise.  The reference configures a single threshold
 * (src/accelerate/token_merger/co_me_2d.py:291-295); a per-frame merge ratio is what the ragged batch-throughput
 * configuration of the benchmark draws.
 */
int come_select_windows_ratios(const void *conf_dev, int dtype, int64_t batch, int64_t frames_per_batch, int grid_h,
                               int grid_w, int group_h, int group_w, const float *ratios_dev, int scope,
                               uint8_t *mask_dev, void *stream);

/*
 * Merge index plan: everything of a merge that depends on the mask only.
 * Replaces block_prefix_scan_kernel + at::cumsum (src/cuda_extension/co_me/src/kernel_token_merge.cu:12-46,
 * 284-286) and the rev_id / weight writes of the scatter kernels (:92-107,146-161,186-190); fallback
 * src/accelerate/token_merger/co_me.py:177-222.
 *   mask_dev          [frames, M] uint8
 *   group_prefix_dev  [frames, M] int32   exclusive scan of (mask ? 1 : G) inside a frame
 *   offsets_dev       [frames + 1] int32  packed start row of every frame; offsets[frames] = P
 *   rev_id_dev        [frames * N] int64  packed row of every input token, in the input token order
 *   weight_dev        [>= P] float32      tokens represented by every packed row (G or 1); a buffer of
 *                                         frames * N floats always suffices
 *   seg_max_dev       [1] int32           longest packed frame (max_seqlen of frame attention); may be NULL
 *   workspace_dev     come_merge_plan_workspace_bytes(frames) bytes of scratch
 */
size_t come_merge_plan_workspace_bytes(int64_t frames);
int come_merge_plan(const uint8_t *mask_dev, int64_t frames, const come_layout_t *layout,
                    int32_t *group_prefix_dev, int32_t *offsets_dev, int64_t *rev_id_dev, float *weight_dev,
                    int32_t *seg_max_dev, void *workspace_dev, size_t workspace_bytes, void *stream);

/*
 * Same plan, for callers that must not allocate device memory and have no workspace to hand over.
 * No counterpart in the reference (its extension allocates freely through the PyTorch allocator).
 *
 * Who needs it: an inference-engine plugin whose enqueue hook runs after the engine has frozen its memory plan,
 * a real-time loop that forbids allocation once it is running, or a host that only owns the tensors it was given.
 * Such a caller still passes every input and output buffer; only the scratch (one int per frame) comes from a
 * fixed array inside the library, so every GPU that loads the library holds COME_MERGE_PLAN_STATIC_MAX_FRAMES ints
 * (16 KiB) for the life of the process.  The function calls no cudaMalloc / cudaFree or other allocating routine.
 *
 *   - frames above COME_MERGE_PLAN_STATIC_MAX_FRAMES are refused with COME_ERR_ARG and a message;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, with
 *     that device current); make that first call before starting any stream capture;
 *   - all calls on a device share the one array, which keeps the previous call's contents (each call overwrites
 *     the part it reads, nothing relies on zeros); two calls whose kernels overlap on the GPU -- different streams
 *     without an ordering between them -- race on it and produce garbage.  Order them, or use come_merge_plan.
 */
#define COME_MERGE_PLAN_STATIC_MAX_FRAMES 4096
int come_merge_plan_static(const uint8_t *mask_dev, int64_t frames, const come_layout_t *layout,
                           int32_t *group_prefix_dev, int32_t *offsets_dev, int64_t *rev_id_dev, float *weight_dev,
                           int32_t *seg_max_dev, void *stream);

/*
 * Merge data movement: packed rows from the token grid.
 * Replaces token_merge_scatter_kernel{_vec4,} + token_merge_special_kernel
 * (src/cuda_extension/co_me/src/kernel_token_merge.cu:50-191) and, for a 2-D layout, the gather pass of
 * func_token_merge_2d (src/accelerate/token_merger/co_me_2d.py:193-211).
 *   tokens_dev [frames, N, channels] contiguous; out_dev [P, channels]; same dtype.
 * A merged window is the float32 left-to-right sum of its G rows divided by G, rounded once to dtype.
 */
int come_merge(const void *tokens_dev, int dtype, int64_t frames, int64_t channels, const come_layout_t *layout,
               const uint8_t *mask_dev, const int32_t *group_prefix_dev, const int32_t *offsets_dev,
               void *out_dev, void *stream);

/*
 * Merge fused with the LayerNorm in front of it: out = merge(LayerNorm_C(tokens)), tokens read once.  Every source row is
 * normalised over its `channels` values (float32 statistics, y = gamma * (x - mean) * rstd + beta, rounded to dtype like
 * the module's output tensor), then merged windows average their normalised rows as come_merge does.  Replaces
 * block.norm1 followed by token_merger.merge of the per-layer mode (src/thirdparty/vggt/layers/block.py:73 ->
 * src/accelerate/vggt/direct.py:97-101).  gamma / beta: [channels] in dtype.  Needs 16-byte aligned pointers, channels a
 * multiple of 16 bytes and at most 256 such vectors (1024 float32 / 2048 16-bit channels), group size <= 9; anything
 * else returns COME_ERR_UNSUPPORTED (run the LayerNorm and come_merge separately).
 */
int come_merge_layernorm(const void *tokens_dev, int dtype, int64_t frames, int64_t channels, const come_layout_t *layout,
                         const void *gamma_dev, const void *beta_dev, float eps, const uint8_t *mask_dev,
                         const int32_t *group_prefix_dev, const int32_t *offsets_dev, void *out_dev, void *stream);

/*
 * Unmerge: out[i, :] = merged[rev_id[i], :].
 * Replaces token_split_gather_kernel{_vec4,} (src/cuda_extension/co_me/src/kernel_token_merge.cu:195-233,
 * host :354-398); fallback index_select (src/accelerate/token_merger/co_me.py:241-254).
 */
int come_unmerge(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels, int dtype,
                 void *out_dev, void *stream);

/*
 * Unmerge into a wider destination: out[i * out_row_stride + c] = merged[rev_id[i], c] for c < channels
 * (out_row_stride in elements, >= channels).  Two calls with out_dev and out_dev + channels write the
 * [frame-block | global-block] concatenation [B, S, N, 2C] of a retained layer in place, which the reference
 * builds from two split() results and a torch.cat (src/accelerate/vggt/fused.py:157-167): one full read and
 * write of the restored tokens less.  With out_row_stride == channels it is come_unmerge.
 */
int come_unmerge_strided(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels, int dtype,
                         void *out_dev, int64_t out_row_stride, void *stream);

/*
 * Unmerge fused with the residual update of a transformer block:
 *   out[i, c] = residual[i, c] + scale[c] * merged[rev_id[i], c]
 * evaluated in the element type like the tensor expression (product rounded, then sum rounded; scale_dev may be NULL
 * = no product).  Replaces split() followed by LayerScale and the residual add of the block the attention sits in
 * (src/accelerate/vggt/direct.py:117-118 -> src/thirdparty/vggt/layers/block.py:73,90 `x + ls1(attn(norm1(x)))`,
 * LayerScale = x * gamma, src/thirdparty/vggt/layers/layer_scale.py:21-22): one pass instead of three over the dense
 * tokens.  out_dev may alias residual_dev (every element is read before it is written by the same thread).
 */
int come_unmerge_residual(const void *merged_dev, const int64_t *rev_id_dev, int64_t total, int64_t channels, int dtype,
                          const void *residual_dev, const void *scale_dev, void *out_dev, void *stream);

/*
 * Residual update of a transformer sub-block fused with the LayerNorm that opens the next one, on packed rows [rows, C]:
 *   x_out  = x + scale * branch          (LayerScale, then the residual add; product rounded, then sum rounded)
 *   normed = LayerNorm(x_out) * gamma + beta   (float32 statistics, result rounded to the element type)
 * i.e. `x = x + ls(branch)` followed by `norm(x)` of the jagged block (src/accelerate/vggt/module/block.py:66-79:
 * `.apply(self.block.ls1)`, `residual_x + attn_x.tokens`, `.apply(self.block.norm2)`; the same pair closes the MLP
 * sub-block and opens the next block's norm1): one read of x and branch and one write of each result instead of three
 * elementwise passes.  Optional parts: branch_dev NULL = LayerNorm of x alone (x_out_dev ignored); scale_dev NULL = no
 * LayerScale; normed_dev NULL = residual update only; x_out_dev NULL = the updated stream is not stored.
 * x_out_dev may alias x_dev and normed_dev may alias branch_dev (a row is read completely before it is written).
 * Channels: a multiple of 16 bytes, at most 4096 bytes per row.
 */
int come_residual_layernorm(const void *x_dev, const void *branch_dev, const void *scale_dev, int64_t rows, int64_t channels,
                            int dtype, const void *gamma_dev, const void *beta_dev, float eps, void *x_out_dev,
                            void *normed_dev, void *stream);

/*
 * Suffix tokens of jagged segments (ITokenMerger.JaggedTokens.add_suffix / split_suffix,
 * src/interface/token_merger.py:23-100; used around the MapAnything blocks, src/accelerate/ma/fused.py:186-214).
 *
 * come_suffix_add: every one of the `segments` segments of the packed tokens [total, channels] (offset int64
 * [segments + 1], weight float32 [total]) is extended by its `suffix_len` rows of suffix [segments, suffix_len, channels],
 * weight 1: out_tokens [total + segments * suffix_len, channels], out_weight, out_offset[m] = offset[m] + m * suffix_len.
 * come_suffix_split: the inverse: the last `suffix_len` rows of every segment go to suffix_out
 * [segments, suffix_len, channels], the rest is packed again; out_offset[m] = offset[m] - m * suffix_len.  The caller
 * checks that every segment holds at least suffix_len rows (the reference raises ValueError after reading the lengths
 * back, token_merger.py:79-83); the library only checks the total.
 * The reference builds both from arange / searchsorted / index_copy_ / index_select: about ten launches and two extra
 * passes over the tokens; here one launch moves every row once.
 */
int come_suffix_add(const void *tokens_dev, const float *weight_dev, const int64_t *offset_dev, int64_t segments,
                    int64_t total, int64_t channels, int dtype, const void *suffix_dev, int64_t suffix_len,
                    void *out_tokens_dev, float *out_weight_dev, int64_t *out_offset_dev, void *stream);
int come_suffix_split(const void *tokens_dev, const float *weight_dev, const int64_t *offset_dev, int64_t segments,
                      int64_t total, int64_t channels, int dtype, int64_t suffix_len, void *out_tokens_dev,
                      float *out_weight_dev, int64_t *out_offset_dev, void *suffix_out_dev, void *stream);

/*
 * Variable-length attention forward with an optional additive per-key bias:
 *   out[s:e, h] = softmax(q[s:e, h] k[s:e, h]^T * softmax_scale + bias[s:e][None, :]) v[s:e, h]
 * for every packed segment [cu_seqlens[i], cu_seqlens[i+1]) and head h; non-causal, no dropout.
 * Replaces varlen_fwd / varlen_fwd_w_perkey_bias (src/cuda_extension/flash_attn/flash_api.cpp:291-599,
 * kernel src/cuda_extension/flash_attn/src/flash_fwd_kernel.h:30-55,80-545).
 *   q/k/v_dev     element (row, head, d) at ptr[row * row_stride + head * head_dim + d] (strides in elements);
 *                 dtype COME_F16 or COME_BF16
 *   bias_dev      [total] in dtype, or NULL
 *   out_dev       [total, num_heads, head_dim] with row stride out_row_stride (elements)
 *   lse_dev       [num_heads, total] float32 log-sum-exp of the biased scaled scores; may be NULL
 *   max_seqlen    upper bound of the segment lengths (sizes the grid only)
 * head_dim 64 runs on the tcgen05 tensor-core kernel; other head dims (multiples of 8 up to 256) run on a
 * plain CUDA-core kernel.  `backend`: 0 = automatic, 1 = force the CUDA-core kernel, 2 = require tcgen05.
 * k and v must be finite in the WHOLE packed buffer: the tensor-core kernel loads the partial last key tile of a segment
 * together with the first rows of the next segment and masks them with probability 0, and 0 x Inf is NaN (rows past
 * `total` are zero-filled by the hardware).
 */
int come_attn_varlen_fwd(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t total,
                         int num_heads, int head_dim, int64_t q_row_stride, int64_t k_row_stride,
                         int64_t v_row_stride, const void *bias_dev, const int32_t *cu_seqlens_dev,
                         int num_segments, int max_seqlen, float softmax_scale, void *out_dev,
                         int64_t out_row_stride, float *lse_dev, int backend, void *stream);

/*
 * The same attention for a slice of the query rows: q / out / lse hold only the global rows
 * [q_row_begin, q_row_begin + q_rows) (lse is [num_heads, q_rows]), k / v / bias / cu_seqlens still describe all
 * `total` packed tokens.  This is the per-GPU piece of global attention sharded by query rows: every GPU attends
 * its own rows to the all-gathered keys and values.  No counterpart in the reference (single GPU only); with
 * q_row_begin = 0 and q_rows = total it is come_attn_varlen_fwd.
 *   max_seqlen_dev  optional (may be NULL): one int32 in device memory, the true longest segment.  max_seqlen (host) must
 *                   still be an upper bound; a caller that cannot read the true value back (a captured graph that
 *                   serves every merge mask) passes its worst case there and the value the plan kernel wrote
 *                   (come_merge_plan's seg_max_dev) here, so that the kernel's work list holds no empty query blocks.
 */
int come_attn_varlen_fwd_rows(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t total,
                              int64_t q_row_begin, int64_t q_rows, int num_heads, int head_dim, int64_t q_row_stride,
                              int64_t k_row_stride, int64_t v_row_stride, const void *bias_dev,
                              const int32_t *cu_seqlens_dev, int num_segments, int max_seqlen,
                              const int32_t *max_seqlen_dev, float softmax_scale, void *out_dev, int64_t out_row_stride,
                              float *lse_dev, int backend, void *stream);

/*
 * Attention of q_rows query rows to ONE set of kv_rows keys / values that need not contain them:
 *   out[i, h] = softmax(q[i, h] k[:, h]^T * softmax_scale + bias[None, :]) v[:, h],   lse[h, i] likewise.
 * No counterpart in the reference (single GPU only).  It is the second half of global attention sharded over GPUs with
 * the exchange hidden behind compute: a GPU first attends its rows to its own keys (come_attn_varlen_fwd) while the other
 * GPUs' keys / values are still in flight, then attends the same rows to the gathered remote keys with this call, and
 * come_attn_combine merges the two results.  Layouts as in come_attn_varlen_fwd; bias_dev [kv_rows] or NULL.
 */
int come_attn_cross_fwd(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t q_rows, int64_t kv_rows,
                        int num_heads, int head_dim, int64_t q_row_stride, int64_t k_row_stride, int64_t v_row_stride,
                        const void *bias_dev, float softmax_scale, void *out_dev, int64_t out_row_stride, float *lse_dev,
                        int backend, void *stream);

/*
 * The tensor-core attention kernel is persistent: one CTA per SM walks the work list, and a CTA takes a whole SM.  A
 * caller that runs a communication kernel next to it (the key / value all-gather of the next step on another stream)
 * leaves that kernel some SMs with this call: the following attention launches OF THE CALLING HOST THREAD use at most
 * max_ctas CTAs (0 = one per SM again).  Without it the attention CTAs that do not fit start only when the other kernel
 * has finished, and the statically divided work list ends late.  No counterpart in the reference.
 */
int come_attn_set_cta_limit(int max_ctas);

/*
 * Exact merge of two attention results of the same query rows over DISJOINT key sets, from their log-sum-exps:
 *   w_x = exp(lse_x - max(lse_a, lse_b));  out = (w_a out_a + w_b out_b) / (w_a + w_b);  lse_out = max + log(w_a + w_b)
 * out_* [rows, num_heads, head_dim] contiguous in dtype (COME_F16 / COME_BF16), lse_* [num_heads, rows] float32;
 * out_dev may alias out_a_dev or out_b_dev, lse_out_dev (may be NULL) may alias lse_a_dev or lse_b_dev.
 * The inputs were rounded to dtype by the two attention launches, so the result differs from a single launch over all
 * keys by that rounding (about 2^-9 relative for bfloat16), not bit for bit.  No counterpart in the reference.
 */
int come_attn_combine(const void *out_a_dev, const float *lse_a_dev, const void *out_b_dev, const float *lse_b_dev,
                      int dtype, int64_t rows, int num_heads, int head_dim, void *out_dev, float *lse_out_dev, void *stream);

/*
 * come_attn_cross_fwd with the keys of every work item split into key_parts shares (1 .. 64, each at least one 64-key tile):
 * for launches with few work items per SM, where the last round of the persistent kernel would run with most SMs idle
 * (448 items on 148 SMs take four rounds; their last block of query rows split nine ways fills one short round instead).
 * Share p attends the query rows to its share of the keys and writes out_parts[p] ([key_parts, q_rows, num_heads, head_dim]
 * contiguous, dtype) and lse_parts[p] ([key_parts, num_heads, q_rows] float32, required); come_attn_combine_parts merges them
 * like come_attn_combine (same rounding remark).  tcgen05 kernel only (head_dim 64), else COME_ERR_UNSUPPORTED.
 * No counterpart in the reference.
 */
int come_attn_cross_fwd_parts(const void *q_dev, const void *k_dev, const void *v_dev, int dtype, int64_t q_rows,
                              int64_t kv_rows, int num_heads, int head_dim, int64_t q_row_stride, int64_t k_row_stride,
                              int64_t v_row_stride, const void *bias_dev, float softmax_scale, int key_parts,
                              void *out_parts_dev, float *lse_parts_dev, int backend, void *stream);
int come_attn_combine_parts(const void *out_parts_dev, const float *lse_parts_dev, int key_parts, int dtype, int64_t rows,
                            int num_heads, int head_dim, void *out_dev, float *lse_out_dev, void *stream);

/*
 * Pre-attention preparation of the packed qkv tensor [total, 3, num_heads, head_dim], in place, one pass:
 *   q, k <- LayerNorm over head_dim (affine gamma / beta; skipped when the four pointers are NULL)
 *   q, k <- 2-D rotary position embedding with integer positions pos[total, 2] = (y, x): the first head_dim/2
 *           features rotate with y, the rest with x (skipped when pos_dev is NULL)
 *   bias_out[i] = log(weight[i]) in dtype (skipped when both are NULL)
 * v is not touched.  Replaces prepare_packed_self_attention_qkv, inference branch
 * (src/accelerate/common/qkv.py:29-39: q_norm, k_norm, rope applied through four full-tensor copies), the rotary
 * module it calls (src/thirdparty/vggt/layers/rope.py:116-187) and the bias expression of the attention module
 * (src/accelerate/vggt/module/bias_attention.py:120).  Arithmetic follows the reference's roundings: statistics and
 * the affine map in float32, the normalised value rounded to dtype, then t*cos, rot(t)*sin and their sum each
 * rounded to dtype.
 *   cos/sin_table_dev  [table_rows, head_dim/2] in dtype: row p = cos / sin of the dtype-rounded angles
 *                      p * base^(-2i/(head_dim/2)), i = 0..head_dim/4-1, repeated twice
 *                      (rope.py:87-114; the caller caches them like the reference does)
 *   gamma / beta       [head_dim] in dtype
 * A position outside [0, table_rows) is clamped and raises bit 16 of the device status word.
 * dtype COME_F16 or COME_BF16; head_dim 32/64/128/256; one CTA of 2*num_heads*head_dim/8 threads handles a row:
 * that count must be a multiple of 32 and <= 512.
 */
int come_qkv_prepare(void *qkv_dev, int dtype, int64_t total, int num_heads, int head_dim, const void *q_gamma_dev,
                     const void *q_beta_dev, const void *k_gamma_dev, const void *k_beta_dev, float eps,
                     const int64_t *pos_dev, const void *cos_table_dev, const void *sin_table_dev, int64_t table_rows,
                     const float *weight_dev, void *bias_out_dev, void *stream);

/*
 * Integer (y, x) positions of the packed rows, pos_out[P, 2] int64, computed from the merge plan alone: special
 * tokens (0, 0), patch (y, x) -> (y + 1, x + 1), a merged window -> the truncated bfloat16 mean of its patches'
 * positions (its centre).  Replaces merging the [B, S, N, 2] bfloat16 position tensor through the token merger and
 * truncating it (src/accelerate/vggt/fused.py:113-129).  2-D layouts only.
 */
int come_packed_positions(const uint8_t *mask_dev, const int64_t *rev_id_dev, int64_t frames,
                          const come_layout_t *layout, int64_t *pos_out_dev, void *stream);

/*
 * Device status word: kernels that wait on hardware barriers give up after a bounded number of polls and
 * record a non-zero code here instead of hanging.  Reads it back (synchronises the device) and optionally
 * clears it.  Returns COME_OK with *value == 0 when no kernel reported a problem, COME_ERR_DEVICE with the word in
 * *value (and a message naming its bits) otherwise.  Bits 0-8: a wait of the attention kernel ran out (while the word is
 * raised, attention launches return at once without touching their outputs); bit 15: the wait self-test below; bit 16: a
 * position outside the rotary table was clamped by come_qkv_prepare; bit 17: a wait of the bulk-copy merge kernel ran out;
 * bit 18: come_peer_wait gave up.
 */
int come_device_status(uint32_t *value, int clear);

/*
 * Self-test of the failure path, for deployments that want to see it work once: a one-CTA kernel waits, with the
 * attention kernel's bounded wait, on a barrier that nothing arrives at; after `ticks` clocks (at most 2^26, a few
 * hundredths of a second) the wait gives up, raises bit 15 of the device status word and the kernel returns normally.
 * waited_dev (may be NULL): one int64 in device memory that receives the clocks waited.  Nothing faults or hangs; clear
 * the word with come_device_status(&v, 1) afterwards.  No counterpart in the reference.
 */
int come_selftest_bounded_wait(int64_t ticks, int64_t *waited_dev, void *stream);

/*
 * Exchange of row blocks between the GPUs of one node through peer-mapped memory (one process per GPU): the transport of
 * the key / value all-gather of a global attention layer whose frames are sharded over the GPUs.  The reference has no
 * multi-GPU inference path; these entry points have no counterpart there.
 *
 *   come_peer_alloc   cudaMalloc of a zeroed "window" on the current device + its CUDA IPC handle (COME_PEER_HANDLE_BYTES
 *                     bytes, to be sent to the other processes by any host channel).
 *   come_peer_open    maps another process's window (its handle) into this process; peer access is enabled lazily.
 *   come_peer_close / come_peer_free   undo the two.
 *   come_peer_copy    one cudaMemcpyAsync(dst, src, bytes) on `stream`; either side may be a mapped peer window: the driver
 *                     moves the bytes over NVLink, no kernel of this library is involved.
 *   come_peer_signal  one small kernel: for every rank p != rank a release store of `value` into word `rank` of p's flag
 *                     array.  peer_flags_dev: device array of `world` pointers, entry p = the address of rank p's flag
 *                     array (world int32 words inside p's window) as mapped in THIS process.
 *   come_peer_wait    one small kernel: returns when every word p != rank of this rank's own flag array has reached `value`
 *                     (written by the peers' come_peer_signal), or after limit_ns nanoseconds (at most 120 s), in which
 *                     case bit 18 of the device status word is raised and the stream simply continues: nothing hangs.
 * Usage per exchange k = 1, 2, ...: copy the local block into the own window (slot k & 1), signal k, wait k, copy the
 * peers' blocks out of their windows.  Two slots suffice: a rank that signals k + 1 has finished its copies of exchange k.
 */
#define COME_PEER_HANDLE_BYTES 64
int come_peer_alloc(int64_t bytes, void **ptr_out, void *handle_out);
int come_peer_open(const void *handle, void **ptr_out);
int come_peer_close(void *ptr);
int come_peer_free(void *ptr);
int come_peer_copy(void *dst, const void *src, int64_t bytes, void *stream);
int come_peer_signal(void *const *peer_flags_dev, int world, int rank, int32_t value, void *stream);
int come_peer_wait(const int32_t *flags_dev, int world, int rank, int32_t value, int64_t limit_ns, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* COME_B200_H */
