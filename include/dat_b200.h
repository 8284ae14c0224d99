/*
 * dat_b200.h — C ABI of the B200-native DA-Transformer custom ops.
 *
 * These entry points are what the reference's pybind module `dag_loss_fn`
 * (fs_plugins/custom_ops/dag_loss.cpp:19-29) exports, re-cut as a plain C
 * boundary: raw device pointers, sizes, element strides, a dtype enum and a CUDA
 * stream; no torch types.  The library allocates nothing: every output and every
 * workspace is provided by the caller.  All work is enqueued on `stream`; no
 * entry point synchronises the host.
 *
 * Every function returns DAT_OK (0) or a DAT_ERR_* code; dat_last_error() gives
 * the message of the calling thread's last failure.
 *
 * Tensors (same meaning as fs_plugins/custom_ops/dag_loss.py:71-100):
 *   match_all [B,T,L] fp32 contiguous     log P(y_t | v_j)
 *   links     [B,L,K] fp32 contiguous     band format, links[b,i,d] = log P(v_i -> v_{i+d+1})
 *   output_length, target_length [B] int64 (device)
 * Sentences whose lengths the reference would trap on (target_length < 2,
 * output_length < 2, output_length < target_length, dag_loss.cu:68-69) or that
 * exceed the padded sizes are "invalid": loss = -inf, zero gradients, path = -1,
 * and bit DAT_STATUS_BAD_LENGTH is OR-ed into *status.
 */
#ifndef DAT_B200_H
#define DAT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DAT_B200_VERSION 100

enum dat_status_code {
    DAT_OK = 0,
    DAT_ERR_BAD_ARG = 1,      /* null pointer, non-positive size, bad stride      */
    DAT_ERR_UNSUPPORTED = 2,  /* dtype / size outside what the kernels implement  */
    DAT_ERR_LAUNCH = 3,       /* CUDA reported an error at launch                 */
    DAT_ERR_NO_DEVICE = 4     /* no usable CUDA device / wrong architecture       */
};

enum dat_dtype {
    DAT_F32 = 0,
    DAT_F16 = 1,
    DAT_BF16 = 2
};

/* bits OR-ed by the kernels into the optional device status word */
#define DAT_STATUS_BAD_LENGTH 1 /* a sentence had invalid lengths                  */
#define DAT_STATUS_NO_PATH 2    /* best alignment: a sentence has no finite path   */
#define DAT_STATUS_BAD_INDEX 4  /* gather: an index outside [0, vocab)             */
#define DAT_STATUS_FAST_FALLBACK 8 /* dat_dag_loss_fast recomputed a sentence exactly (informational) */

int dat_version(void);
const char *dat_last_error(void);
const char *dat_status_string(int code);

/* Bytes of the fp64 workspace `offsets` of dat_dag_loss for a batch. */
size_t dat_dag_loss_offsets_bytes(int bsz, int tarlen);
/* Bytes of the workspace of dat_dag_best_alignment for a batch. */
size_t dat_dag_best_alignment_workspace_bytes(int bsz, int tarlen, int prelen);

/*
 * Replaces `logsoftmax_gather` (dag_loss.cpp:22; logsoftmax_gather.cu:313-377).
 *   selected_result[b,l,s] = log_softmax(word_ins_out[b,l,:])[select_idx[b,l,s]]   (fp32)
 * word_ins_out [bsz,prelen,vocab] contiguous, dtype DAT_F32/F16/BF16; it is only READ
 * (the reference overwrites it with probabilities when a gradient is needed; here the
 * two row statistics written to `row_stats` [bsz*prelen,2] = (max, log sum exp(x-max))
 * carry what the backward needs; pass NULL when no gradient is needed).
 * select_idx and selected_result are addressed through ELEMENT strides, so the
 * stride-(S,0,1) expand the criterion passes (nat_dag_loss.py:168) and a
 * [B,S,L]-contiguous result can be used directly.
 */
int dat_logsoftmax_gather(const void *word_ins_out, int dtype,
                          const int64_t *select_idx, int64_t idx_stride_b, int64_t idx_stride_l,
                          int64_t idx_stride_s,
                          float *selected_result, int64_t sel_stride_b, int64_t sel_stride_l,
                          int64_t sel_stride_s,
                          float *row_stats, int32_t *status,
                          int bsz, int prelen, int slen, int vocab, void *stream);

/*
 * Replaces the Python backward of DagLogsoftmaxGatherFunc (dag_loss.py:217-231:
 * probs.mul_(-sum_s g) then scatter_add_(idx, g)).  IN PLACE: word_ins_out holds the
 * logits on entry and the dense gradient (same dtype, fp32 math, rounded once) on
 * return:  d[b,l,v] = -softmax(x[b,l,:])[v] * sum_s g[b,l,s] + sum_{s: idx=v} g[b,l,s].
 * slen <= 4096.
 */
int dat_logsoftmax_gather_backward(void *word_ins_out, int dtype,
                                   const int64_t *select_idx, int64_t idx_stride_b,
                                   int64_t idx_stride_l, int64_t idx_stride_s,
                                   const float *grad_selected, int64_t g_stride_b,
                                   int64_t g_stride_l, int64_t g_stride_s,
                                   const float *row_stats,
                                   int bsz, int prelen, int slen, int vocab, void *stream);

/*
 * dat_logsoftmax_gather with two pieces of the criterion's glue done in the same pass over the
 * logits (what surrounds the call at fs_plugins/criterions/nat_dag_loss.py:246-262 and 166-179):
 *   argmax (optional, [bsz*prelen] int64): word_ins_out.argmax(-1), the glancing sampler's
 *     prediction (nat_dag_loss.py:246), with torch.argmax's result on ties (first index) and NaN;
 *   force_emit (optional, [bsz,prelen] int64 contiguous, -1 = free): the forced alignment of
 *     NATDAGLoss._force_aligment (nat_dag_loss.py:111-120) applied to the gathered values, which
 *     must then be the match matrix (slen = tarlen, select_idx = the target tokens): for every
 *     target step s that some vertex of the sentence is forced to emit, selected_result[b,l,s] is 0
 *     at the forced vertex and -inf elsewhere.  forced_step ([bsz,slen] int32, written here) marks
 *     those steps; dat_logsoftmax_gather_backward_fused takes it to stop the gradient there, as the
 *     reference's masked_fill does.  A forced step >= slen sets DAT_STATUS_BAD_INDEX.
 * slen <= 8192 when force_emit is given.
 */
int dat_logsoftmax_gather_fused(const void *word_ins_out, int dtype,
                                const int64_t *select_idx, int64_t idx_stride_b, int64_t idx_stride_l,
                                int64_t idx_stride_s,
                                float *selected_result, int64_t sel_stride_b, int64_t sel_stride_l,
                                int64_t sel_stride_s,
                                float *row_stats, int64_t *argmax, const int64_t *force_emit,
                                int32_t *forced_step, int32_t *status,
                                int bsz, int prelen, int slen, int vocab, void *stream);

/* dat_logsoftmax_gather_backward for a forward done with force_emit: gradients arriving at the
 * forced steps (forced_step[b,s] != 0) are dropped (nat_dag_loss.py:117).  forced_step may be NULL. */
int dat_logsoftmax_gather_backward_fused(void *word_ins_out, int dtype,
                                         const int64_t *select_idx, int64_t idx_stride_b,
                                         int64_t idx_stride_l, int64_t idx_stride_s,
                                         const float *grad_selected, int64_t g_stride_b,
                                         int64_t g_stride_l, int64_t g_stride_s,
                                         const float *row_stats, const int32_t *forced_step,
                                         int bsz, int prelen, int slen, int vocab, void *stream);

/*
 * Replaces `dag_loss` (dag_loss.cpp:19; dag_loss.cu:313-375).
 * Runs the alpha recursion and, if require_gradient, the beta recursion, and writes
 * loss[b] = log P(target | graph) (beta[b,0,0] when require_gradient, else
 * alpha[b,tl-1,ol-1], as dag_loss.py:106-109 picks them).
 * alpha, beta: caller-provided fp32 workspaces [bsz,tarlen,prelen] consumed by
 * dat_dag_loss_backward (beta may be NULL when !require_gradient).  They hold the
 * recursion rows in the log2 domain, each row shifted by a per-row offset kept in the
 * fp64 workspace `offsets` (dat_dag_loss_offsets_bytes); only the reachable window
 * j in [t, t + ol - tl] of each row t < tl is written.
 * config: accepted for compatibility with DagLossFunc.config, ignored.
 * Limits (checked before anything is launched, DAT_ERR_UNSUPPORTED with the limit in the message; the
 * same for dat_dag_loss_fast and dat_dag_loss_static): prelen <= 2048, and tarlen <= 7168 when a
 * gradient is wanted (the exact backward keeps one column of all steps in shared memory).
 */
int dat_dag_loss(const float *match_all, const float *links, const int64_t *output_length,
                 const int64_t *target_length, int require_gradient,
                 float *alpha, float *beta, double *offsets, float *loss, int32_t *status,
                 int bsz, int tarlen, int prelen, int translen, int config, void *stream);

/*
 * Fast path of `dag_loss` with require_gradient (replaces the same reference function as
 * dat_dag_loss: dag_loss.cpp:19; dag_loss.cu:313-375).  Same outputs and the same workspace
 * format as dat_dag_loss(..., require_gradient = 1, ...), so dat_dag_loss_backward consumes them
 * unchanged.  The recursions run in the probability domain on E = exp(links), each link
 * exponentiated once per sweep instead of once per target step.  `scratch`
 * (dat_dag_loss_fast_scratch_bytes bytes for the current device, caller-allocated, contents
 * irrelevant on entry) holds what dat_dag_loss_backward_fast reuses: the per-sentence flags and
 * row maxima and, for sentences too large to keep their rows in shared memory, a square copy
 * of E.  Power-of-two rescaling keeps ~160 binades below the largest term; an a-posteriori bound on the mass that
 * could have been flushed decides per sentence whether the result is kept or the sentence is
 * recomputed by the exact log-domain kernel inside the same call, so the result always meets
 * the tolerances of dat_dag_loss.
 */
size_t dat_dag_loss_fast_scratch_bytes(int bsz, int tarlen, int prelen);
int dat_dag_loss_fast(const float *match_all, const float *links, const int64_t *output_length,
                      const int64_t *target_length, float *alpha, float *beta, double *offsets,
                      float *loss, int32_t *status, void *scratch,
                      int bsz, int tarlen, int prelen, int translen, void *stream);

/* What the dynamic-range check of the last dat_dag_loss_fast call on `scratch` decided, as two device
 * words: count[0] = sentences recomputed by the exact kernels (what the status bit
 * DAT_STATUS_FAST_FALLBACK summarises), count[1] = sentences whose forward was kept but whose
 * grad_links will come from the exact kernel.  No counterpart in the reference. */
int dat_dag_loss_fast_flagged(const void *scratch, int32_t *count, int bsz, int tarlen, int prelen,
                              void *stream);

/*
 * Backward for a forward done by dat_dag_loss_fast (replaces dag_loss_backward, dag_loss.cpp:20;
 * dag_loss.cu:518-571, like dat_dag_loss_backward).  `scratch` is the forward's scratch,
 * untouched since (the call writes its own working data into it: it is declared const because its
 * size and meaning for the caller do not change).  grad_links is computed in product form (one exp per
 * stored row entry, then a matrix product over the target steps on the tensor cores) for the
 * sentences that passed the forward's dynamic-range check and by the exact kernel for the others.
 */
int dat_dag_loss_backward_fast(const float *grad_output, const float *alpha, const float *beta,
                               const double *offsets, const float *match_all, const float *links,
                               const int64_t *output_length, const int64_t *target_length,
                               float *grad_match_all, float *grad_links, const void *scratch,
                               int bsz, int tarlen, int prelen, int translen, void *stream);

/*
 * No counterpart in the reference.  Same result as dat_dag_loss(..., require_gradient = 0):
 * loss[b] = log P(target | graph), but the recursion workspace is a fixed array inside the
 * library image instead of caller memory, and the call allocates nothing (no cudaMalloc,
 * no allocating library routine).  It exists for hosts that cannot obtain device memory at
 * call time: a serving process that gave the whole GPU to its own pool when it started, or a
 * plugin slot whose contract forbids allocation because cudaMalloc synchronises the device
 * and would stall the other streams of the process.  Such a host passes only its inputs and
 * the [bsz] output.
 * Limits: bsz*tarlen*prelen <= 2^21 floats (8 MiB) and bsz*(2*tarlen+2) <= 2^16; beyond
 * that the call fails with DAT_ERR_UNSUPPORTED and a message naming both numbers.  Every GPU
 * that loads the library holds the 8.5 MiB until the process exits.
 * The first call on a device looks up the array's device address (once per device, with that
 * device current); make that first call outside any stream capture.
 * All calls on a device share the one workspace: calls whose kernels overlap on the GPU
 * (different streams) race on it.  Nothing in it has to be cleared between calls.
 */
int dat_dag_loss_static(const float *match_all, const float *links,
                        const int64_t *output_length, const int64_t *target_length,
                        float *loss, int32_t *status,
                        int bsz, int tarlen, int prelen, int translen, void *stream);

/*
 * Replaces `dag_loss_backward` (dag_loss.cpp:20; dag_loss.cu:518-571).
 *   grad_match_all[b,t,j] = g[b] * exp(alpha+beta-match-Z)        (0 where match or Z is +-inf)
 *   grad_links[b,i,d]     = g[b] * sum_t exp(alpha[t,i]+beta[t+1,i+d+1]+links[i,d]-Z)
 * Both outputs are written completely (zeros outside the reachable region).
 * config1/config2: accepted for compatibility, ignored.
 */
int dat_dag_loss_backward(const float *grad_output, const float *alpha, const float *beta,
                          const double *offsets, const float *match_all, const float *links,
                          const int64_t *output_length, const int64_t *target_length,
                          float *grad_match_all, float *grad_links,
                          int bsz, int tarlen, int prelen, int translen, int config1, int config2,
                          void *stream);

/*
 * Replaces `dag_best_alignment` (dag_loss.cpp:21; dag_best_alignment.cu:219-263) and the
 * int32->int64 cast of dag_loss.py:162.
 *   path[b,j] = t if vertex j emits target token t on the max-probability path, else -1.
 * Ties are broken exactly as the reference kernel does for TRANS_BLOCK_SIZE lanes
 * (config 1,2,3,4 -> 4,8,16,32 lanes; dag_best_alignment.cu:253-256): among equal
 * candidates the merge tree prefers lanes in bit-reversed order, then the smaller d.
 * workspace: dat_dag_best_alignment_workspace_bytes(...) bytes, 16-byte aligned.
 * max_score (optional, [bsz] fp32): alpha[b,tl-1,ol-1] of the max-plus recursion.
 */
int dat_dag_best_alignment(const float *match_all, const float *links,
                           const int64_t *output_length, const int64_t *target_length,
                           int64_t *path, float *max_score, void *workspace, int32_t *status,
                           int bsz, int tarlen, int prelen, int translen, int config,
                           void *stream);

/*
 * Per-shard statistics of the criterion in one launch (replaces the elementwise and reduction
 * launches of fs_plugins/criterions/nat_dag_loss.py:190-194 that follow dag_loss, and produces the
 * fp64 buffer the reference all-reduces, fairseq/distributed/utils.py:634-680):
 *   stats[0] = sum_b loss_b / target_length_b over the sentences whose loss is finite,
 *   stats[1] = sum_b target_length_b, stats[2] = bsz, stats[3] = number of sentences with inf/nan loss.
 * loss: [bsz] fp32, target_length: [bsz] int64, stats: [4] fp64, all on the device.
 */
int dat_sentence_stats(const float *loss, const int64_t *target_length, double *stats, int bsz,
                       void *stream);

/*
 * dat_sentence_stats plus the criterion's differentiable scalar (nat_dag_loss.py:190-194) in the same
 * launch: *mean_out = -(1/bsz) * sum_b clean_b / target_length_b (inf/nan sentences zeroed), and
 * grad_scale[b] = d mean / d loss_b = -1 / (target_length_b * bsz), 0 for the zeroed sentences.
 * mean_out: one device float; grad_scale: [bsz] fp32.
 */
int dat_sentence_mean(const float *loss, const int64_t *target_length, double *stats, float *mean_out,
                      float *grad_scale, int bsz, void *stream);

/*
 * Replaces the tail of GlatDecomposedLink.extract_links
 * (fs_plugins/models/glat_decomposed_with_link.py:380-404 with extract_valid_links :319-335): from the
 * per-head transition scores and the per-vertex head log-probabilities to the band links dag_loss
 * reads, without the [B,L,K,H] intermediates of the reference.
 *   content   [bsz,prelen,prelen,heads] fp32 contiguous   log_multi_content (q.k / sqrt(d) per head)
 *   log_gates [bsz,prelen,heads] fp32                     log_softmax of the gate scores
 *   links[b,i,d] = logsumexp_h( log_softmax over the valid successors j of content[b,i,j,h] + log_gates[b,i,h] )
 *                  with j = i+d+1; -inf where j is not a valid successor and for vertices without one.
 * Valid successors of i: i < j <= min(prelen-1, i+translen), and j <= bound_end[b,i] when bound_end
 * ([bsz,prelen] int64, the decoding mask, :390-393) is given, and nonpad[b,j] != 0 when nonpad
 * ([bsz,prelen] uint8, prev_output_tokens != pad, the training mask, :394-395) is given; either may be NULL.
 * head_lse (optional output, [bsz,prelen,heads] fp32): the per-head log-sum-exp the backward needs.
 * heads <= 256; (prelen-1)*heads*4 bytes must fit in shared memory (about 220 KB).
 */
int dat_links_from_heads(const float *content, const float *log_gates, const int64_t *bound_end,
                         const unsigned char *nonpad, float *links, float *head_lse,
                         int bsz, int prelen, int heads, int translen, void *stream);

/*
 * Gradient of dat_links_from_heads (the reference differentiates :380-404 by autograd).
 * grad_content [bsz,prelen,prelen,heads] is written completely (zeros outside the valid successors)
 * and may alias content; grad_log_gates [bsz,prelen,heads].  links / head_lse: the forward's outputs.
 */
int dat_links_from_heads_backward(const float *grad_links, const float *content, const float *log_gates,
                                  const float *links, const float *head_lse, const int64_t *bound_end,
                                  const unsigned char *nonpad, float *grad_content, float *grad_log_gates,
                                  int bsz, int prelen, int heads, int translen, void *stream);

/*
 * Node-passing probabilities of GlatDecomposedLink._analyze_graph
 * (fs_plugins/models/glat_decomposed_with_link.py:559-569): node_pass[b,j] = probability that a path
 * starting at vertex 0 visits vertex j.  links_square [bsz,prelen,prelen] fp32 holds log P(i -> j) and
 * must be -inf on and below the diagonal (what restore_valid_links produces, :337-349).
 */
int dat_node_passing_prob(const float *links_square, float *node_pass, int bsz, int prelen, void *stream);

/*
 * Replaces GlatDecomposedLink.inference_viterbi (fs_plugins/models/glat_decomposed_with_link.py:720-777).
 *   links_square     [bsz,prelen,prelen] fp32  log P(i -> j)  (only read; the reference adds the token
 *                    scores into row 0 in place, :727-732, which changes no result while links[0][0] = -inf)
 *   unreduced_logits [bsz,prelen] fp32, unreduced_tokens [bsz,prelen] int64: max and arg-max over the
 *                    vocabulary of the normalised logits (:721)
 *   joint            != 0 for decode_strategy "jointviterbi" (token scores join every step)
 *   max_length       number of lengths tried (the reference uses 2 * prelen / upsample_scale, :735)
 *   beta             exponent of the length penalty (decode_viterbibeta, :753)
 * Outputs: out_tokens [bsz,max_length] int64, the collapsed token sequence padded with pad_index
 * (repeated and pad tokens dropped as in :762-769); out_length [bsz] its length; out_vertices
 * [bsz,max_length] the vertices of the best path before the collapse (-1 padded); out_score [bsz] the
 * length-normalised score.  Maxima resolve ties to the first index like torch.max.
 * workspace: dat_viterbi_decode_workspace_bytes(...) bytes (per step the back-pointers or the row's values).  prelen <= 4096.
 */
size_t dat_viterbi_decode_workspace_bytes(int bsz, int prelen, int max_length);
int dat_viterbi_decode(const float *links_square, const float *unreduced_logits,
                       const int64_t *unreduced_tokens, const int64_t *output_length, void *workspace,
                       int64_t *out_tokens, int64_t *out_length, int64_t *out_vertices, float *out_score,
                       int32_t *status, int bsz, int prelen, int max_length, int joint, float beta,
                       int64_t pad_index, void *stream);

/*
 * Host-to-device copy of band links [bsz,prelen,translen] that skips the padding (no counterpart in the
 * reference, whose callers keep the links on the device): row i of a graph with n vertices has n-1-i
 * real entries, the rest is -inf that no entry point of this library reads.  Moves, for all sentences,
 * the entries a graph of max_output_length vertices can have; the other bytes of dev_links are left as
 * they are (give or take a few bytes of padding next to the real entries).  Page-locked host memory
 * (cudaHostAlloc / cudaHostRegister, 16-byte aligned) is read directly by a kernel on `stream`, row by
 * row, except the first dat_upload_links_head_rows rows of every sentence (those with at least three
 * quarters of translen real entries), which go whole through the copy engine on a helper stream of the
 * library at the same time (the call's stream waits for both; while `stream` is being captured the kernel
 * moves everything); pageable memory goes through strided copies of 32-row blocks, each cut at its
 * longest row.
 * dat_upload_links_bytes: an upper bound of the bytes the pageable form moves over the bus (the
 * staircase's count).  The page-locked form moves head_rows * translen floats per sentence plus the
 * exact prefixes of the other rows, each rounded to 16 bytes.
 */
size_t dat_upload_links_bytes(int bsz, int prelen, int translen, int max_output_length);
int dat_upload_links_head_rows(int prelen, int translen, int max_output_length);
int dat_upload_links(const float *host_links, float *dev_links, int bsz, int prelen, int translen,
                     int max_output_length, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DAT_B200_H */
