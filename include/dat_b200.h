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

/*
 * Backward for a forward done by dat_dag_loss_fast (replaces dag_loss_backward, dag_loss.cpp:20;
 * dag_loss.cu:518-571, like dat_dag_loss_backward).  `scratch` is the forward's scratch,
 * untouched since.  grad_links is computed in product form (one exp per stored row entry, then
 * a small matrix product over the target steps) for the sentences that passed the forward's
 * dynamic-range check and by the exact kernel for the others.
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
 * Measurement helper, no counterpart in the reference: launches `blocks` CTAs of 1024
 * threads that each execute 8*iters dependent-chain ex2 evaluations per thread, so that
 * blocks*1024*8*iters / elapsed is the device's sustained special-function rate (the
 * roofline denominator of the DAG recursion kernels).  `sink` is one device float.
 */
int dat_probe_mufu(int iters, int blocks, float *sink, void *stream);

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

#ifdef __cplusplus
}
#endif
#endif /* DAT_B200_H */
