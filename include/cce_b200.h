/*
 * cce_b200 — C ABI of the B200 (sm_100a) Cut Cross-Entropy kernels.
 *
 * The reference (apple/ml-cross-entropy) has no FFI: its Python autograd
 * function calls three Triton launchers.  Each entry point below replaces one
 * of those launchers and is what a binding for this path would call:
 *
 *   cce_b200_lse_forward      <- cut_cross_entropy/cce_lse_forward.py:163-237
 *                                (cce_lse_forward_kernel)
 *   cce_b200_indexed_neg_dot  <- cut_cross_entropy/indexed_dot.py:102-158
 *                                (indexed_neg_dot_forward_kernel)
 *   cce_b200_backward         <- cut_cross_entropy/cce_backward.py:346-521
 *                                (cce_backward_kernel)
 *   cce_b200_valid_rows       <- cut_cross_entropy/utils.py:28-49
 *                                (_build_flat_valids, the list of rows the three
 *                                launchers above take as `valids`)
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; the library
 *     never allocates or frees device memory: outputs and workspace belong to
 *     the caller (query the *_workspace_bytes functions first);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it
 *     and the call returns without synchronising;
 *   - return value 0 = success, negative = error (see cce_b200_strerror).
 *     Nothing throws, traps or aborts;
 *   - the first 4 bytes of every workspace are a device status word that the
 *     kernels set to a non-zero code if a bounded wait inside a kernel gave
 *     up.  cce_b200_read_status copies it to the host (synchronises).
 */
#ifndef CCE_B200_H_
#define CCE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of e / c (and of the gradient outputs) */
enum { CCE_DT_F16 = 0, CCE_DT_BF16 = 1, CCE_DT_F32 = 2 };
/* index types of `valids` */
enum { CCE_IDX_I32 = 0, CCE_IDX_I64 = 1 };

/* error codes */
enum {
    CCE_OK = 0,
    CCE_ERR_ARG = -1,        /* null pointer, negative size, unsupported dtype */
    CCE_ERR_ALIGN = -2,      /* a pointer or stride is not aligned as documented */
    CCE_ERR_WORKSPACE = -3,  /* workspace too small */
    CCE_ERR_CUDA = -4,       /* a CUDA runtime/driver call failed (see cce_b200_last_cuda_error) */
    CCE_ERR_DEVICE = -5,     /* not an sm_100 device */
    CCE_ERR_KERNEL_WAIT = -6, /* status word non-zero: a kernel abandoned a bounded wait */
    CCE_ERR_TOO_LARGE = -7,   /* problem needs more scratch than the fixed buffer of cce_b200_lse_forward_static */
    CCE_ERR_UNSUPPORTED = -8  /* feature not compiled into this build (wait tracing needs -DCCE_TRACE=1) */
};

/* Shape and operand description shared by the three entry points.
 * Rows of `e` that take part are listed by `valids` (n_rows entries, indices
 * into the flat [n_total, D] matrix); valids == NULL means rows 0..n_rows-1. */
typedef struct cce_b200_operands {
    const void* e;        /* [n_total, D], row stride lde elements, unit column stride */
    const void* c;        /* [V, D], row stride ldc elements, unit column stride */
    const void* bias;     /* [V] or NULL */
    const void* valids;   /* [n_rows] int32/int64 or NULL */
    int64_t n_total;      /* rows of e (and entries of targets) */
    int64_t n_rows;       /* rows that enter the loss ("B" in the reference) */
    int64_t V;            /* classifier rows held by this rank */
    int64_t D;            /* hidden size */
    int64_t lde, ldc;     /* row strides in elements */
    int32_t dtype;        /* type of e and c: CCE_DT_BF16, CCE_DT_F16, or CCE_DT_F32 (computed as a
                             three-term bf16 split, ~2^-16 relative error per product, 3x the work) */
    int32_t bias_dtype;   /* CCE_DT_* of bias */
    int32_t valids_dtype; /* CCE_IDX_* */
    int32_t has_softcap;  /* 0/1 */
    float softcap;
    /* Optional: the number of rows that enter the loss, kept on the DEVICE (one int64, for instance
     * the count_out of cce_b200_valid_rows in device memory) by a caller that does not want to read
     * it back.  When set, `valids` must be given, n_rows is only an upper bound of the count (buffers
     * and launches are sized for it; n_total is always one) and every kernel takes the real count
     * from here: outputs are written for the first *n_rows_dev rows only.  NULL: n_rows is the count. */
    const int64_t* n_rows_dev;
} cce_b200_operands;

/* lse[i] = log sum_v exp(softcap(e[row_i] . c[v] + bias[v])), i < n_rows.
 * Replaces cce_lse_forward_kernel (cut_cross_entropy/cce_lse_forward.py:163). */
size_t cce_b200_lse_workspace_bytes(const cce_b200_operands* op);
int cce_b200_lse_forward(const cce_b200_operands* op, float* lse /* [n_rows] */,
                         float* tile_max /* [cce_b200_tile_max_elems(op)] or NULL */,
                         void* workspace, size_t workspace_bytes, void* stream);
/* Optional by-product of the forward for a filtered backward: the largest logit (in log2 units)
 * of every (32-row group, 256-column tile) block, [4*ceil(n_rows/128)][ceil(V/256)] floats.
 * Given to cce_b200_backward it lets the backward skip the recomputation of tiles in which every
 * softmax value is provably below filter_eps and no label falls.  (The reference keeps a
 * different by-product for its filter, the mean logit per column, cce_lse_forward.py:95-97.) */
size_t cce_b200_tile_max_elems(const cce_b200_operands* op);
/* Where cce_b200_lse_forward leaves its staged copy of e (the listed rows gathered into a dense
 * [n_rows][pitch] 16-bit matrix, zero padded; made when `valids` is given or TMA cannot address e
 * as it is): returns 1 and the byte offset inside the workspace and the row pitch in elements, 0 if
 * the call stages nothing, negative on bad arguments.  A caller that keeps the forward's workspace
 * alive can hand the copy to cce_b200_backward (e_packed), which then skips making its own. */
int cce_b200_lse_packed_e(const cce_b200_operands* op, size_t* offset, int64_t* pitch);
/* cce_b200_lse_forward with one more optional by-product: col_max_key [V] int32, the largest logit
 * (log2 units) of every vocabulary entry over all rows, stored as an order-preserving integer key
 * (a float f >= 0 as its bit pattern, f < 0 as its bit pattern with the low 31 bits inverted), so
 * that an integer sort of the keys sorts the maxima.  cce_b200_backward uses it, with a vocabulary
 * order, to bound the softmax values of reordered tiles. */
int cce_b200_lse_forward_ex(const cce_b200_operands* op, float* lse, float* tile_max, int32_t* col_max_key,
                            void* workspace, size_t workspace_bytes, void* stream);

/* The reference's ordering key (cut_cross_entropy/cce_lse_forward.py:95-97, the optional
 * `logit_avg` result of its forward kernel): out[v] = softcap(mean_i(e[row_i]) . c[v] + bias[v]).
 * Without soft-capping this is the mean over the rows of the logits of column v, which is what the
 * reference accumulates; with soft-capping it is the soft-cap of the mean of the uncapped logits
 * (monotone in it, so it sorts the vocabulary the same way; the reference averages after capping).
 * Three HBM-bound launches (column means of the listed rows of e, then one warp per row of c),
 * summed in a fixed order. */
size_t cce_b200_logit_avg_workspace_bytes(const cce_b200_operands* op);
int cce_b200_logit_avg(const cce_b200_operands* op, float* out /* [V] */, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Same result as cce_b200_lse_forward, for callers that cannot hand over a workspace.
 * (No counterpart in the reference, whose launcher allocates its own buffers through PyTorch.)
 *
 * Who needs it: a host program that binds this library without a device allocator of its own
 * (a thin FFI caller in another language), a process in which another component has reserved
 * all device memory so that a new driver allocation would fail, or a latency-critical loop that
 * must not hit the implicit device-wide synchronisation of cudaMalloc/cudaFree.  This entry
 * point calls no cudaMalloc, no cudaFree and no allocating library routine: its scratch memory
 * is a fixed array of CCE_B200_STATIC_SCRATCH_BYTES bytes that lives inside the library image on
 * every GPU that loads the library, until the process exits.  The caller passes only the inputs
 * and the output.
 *
 * Limits and rules:
 *  - the scratch the problem needs (what cce_b200_lse_workspace_bytes reports: the per-band
 *    partial sums, plus staged copies when `valids` is given or the operands are not 16-byte
 *    aligned) must fit in the array; otherwise nothing runs and CCE_ERR_TOO_LARGE is returned.
 *    Aligned, dense operands of the Gemma-2-2B head shape (8192 x 2304 against 256000 rows) need
 *    about 4 MiB;
 *  - the first call on each device looks up the device address of the array (with that device
 *    current).  Make that first call outside any stream capture;
 *  - all calls on a device share the one array and it keeps the previous call's contents (the
 *    status word at its start is cleared by every call, everything else that is read is first
 *    written by the same call).  Two calls that overlap on the GPU (different streams, or
 *    different host threads without ordering) race on it: order them. */
#define CCE_B200_STATIC_SCRATCH_BYTES (8u << 20)
int cce_b200_lse_forward_static(const cce_b200_operands* op, float* lse /* [n_rows] */, void* stream);

/* out[i] = -softcap(e[row_i] . c[t] + bias[t]), t = targets[row_i + shift] - vocab_start;
 * rows whose t falls outside [0, V) get 0 (vocab-parallel ranks that do not
 * own the target).  No workspace.
 * Replaces indexed_neg_dot_forward_kernel (cut_cross_entropy/indexed_dot.py:102). */
int cce_b200_indexed_neg_dot(const cce_b200_operands* op, const int64_t* targets /* [n_total] */,
                             int64_t shift, int64_t vocab_start, float* out /* [n_rows] */,
                             void* stream);

/* Tail of the forward pass, one launch: merge the per-rank statistics, form the negative
 * log-likelihood of every row, and reduce or scatter it.
 *   stats [world][2][n_rows] fp32: for each vocabulary shard (rank) the log-sum-exp of every row over
 *   that shard (what cce_b200_lse_forward wrote) and minus the correct-token logit (what
 *   cce_b200_indexed_neg_dot wrote; 0 on ranks that do not own the label).  world = 1 without
 *   vocab parallelism; with it, the block is what an all-gather of the ranks' [2][n_rows] blocks gives.
 *   lse_i = logsumexp_r stats[r][0][i];  nll_i = lse_i + sum_r stats[r][1][i].
 *   reduction 0 (mean) / 1 (sum): loss_out[0] = mean / sum over rows of nll, summed in a fixed order;
 *   reduction 2 (none): loss_out [n_total] receives nll_i at position rows[i] + shift (i when rows is
 *   NULL) and 0 elsewhere.  lse_rows (optional, [n_rows]) receives lse_i (the vector the backward
 *   takes); lse_scatter (optional, [n_total]) receives lse_i at the same positions as the loss, 0 elsewhere.
 *   status_workspace (optional): the workspace of the cce_b200_lse_forward call that produced the
 *   statistics; if its status word is non-zero (a kernel abandoned a wait) every output is NaN.
 *   n_rows_dev (optional): the row count on the device, as in cce_b200_operands; n_rows is then the
 *   upper bound the statistics block is laid out for, and `rows` must be given.
 * Replaces, in cut_cross_entropy/cce.py:139-160 and utils.py:52-61, the element-wise add, the
 * mean/sum and the index-put of handle_reduction_none, and vocab_parallel/utils.py:47-65's merges. */
int cce_b200_loss_tail(const float* stats, int32_t world, int64_t n_rows, const void* rows, int32_t rows_dtype,
                       int64_t shift, int64_t n_total, int32_t reduction, float* lse_rows, float* loss_out,
                       float* lse_scatter, const void* status_workspace, const int64_t* n_rows_dev, void* stream);

/* The rows of the flattened embedding matrix that enter the loss, in ascending order:
 * row r (0 <= r < n_total) is paired with label targets[r + shift] and is listed when that label
 * lies in the same sequence (r % seq_len < seq_len - shift) and differs from ignore_index.
 * rows_out (int32 or int64 by rows_dtype, room for n_total entries) receives the list and
 * count_out[0] (an int64 the device can write: device memory, or pinned host memory, which kernels
 * reach through unified addressing and which spares the read-back a copy-engine transfer that
 * could queue behind a bulk download) its length; the caller waits for the stream, reads the
 * count (the one host synchronisation of the forward pass) and passes rows_out/count on as
 * `valids`/`n_rows`.
 * n_total must be a multiple of seq_len.  Two small launches, no atomics: the list is
 * deterministic; its workspace carries no status word (these kernels never wait).  Replaces
 * (cut_cross_entropy/utils.py:28-49), which the reference evaluates with
 * torch.nonzero / boolean indexing. */
size_t cce_b200_valid_rows_workspace_bytes(int64_t n_total);
int cce_b200_valid_rows(const int64_t* targets /* [n_total] */, int64_t n_total, int64_t seq_len,
                        int64_t shift, int64_t ignore_index, void* rows_out, int rows_dtype,
                        int64_t* count_out, void* workspace, size_t workspace_bytes, void* stream);

typedef struct cce_b200_backward_args {
    cce_b200_operands op;
    const float* lse;        /* [n_rows] full (all-rank) log-sum-exp */
    const int64_t* targets;  /* [n_total]; entry row_i + shift is the label of row_i */
    int64_t shift;
    int64_t vocab_start;     /* first vocabulary index held by this rank (0 without vocab parallelism) */
    const float* d_out;      /* upstream gradient of the loss: 1 element, or [n_total] indexed at row_i + shift */
    int64_t d_out_numel;     /* 1 or n_total */
    const float* d_lse;      /* upstream gradient of the returned lse, [n_total] indexed at row_i + shift, or NULL */
    float grad_scale;        /* 1/n_rows for reduction=mean, else 1 */
    int32_t grad_scale_by_inv_rows; /* 1: multiply grad_scale by 1/(row count) on the device (reduction=mean
                                        when the count lives in op.n_rows_dev); 0 otherwise */
    int32_t has_filter;      /* 0: exact gradient; 1: skip tiles whose |softmax - onehot| < filter_eps everywhere */
    float filter_eps;
    int32_t filter_e;        /* apply the filter to the dE product */
    int32_t filter_c;        /* apply the filter to the dC product */
    void* d_e;               /* [n_total, D] in op.dtype, row stride D, or NULL; fully written (zeros at rows not in valids) */
    int32_t d_e_f32;         /* element type of d_e: 0 = op.dtype, 1 = fp32 (for a caller that reduces dE across ranks in fp32) */
    void* d_c;               /* [V, D] in op.dtype (fp32 for fp32 operands), row stride D, or NULL */
    float* d_bias;           /* [V] fp32 or NULL */
    const float* tile_max;   /* by-product of cce_b200_lse_forward for the same operands, or NULL */
    /* Optional vocabulary ordering (the reference's `vocab_ordering`, cce_backward.py:154-155): a
     * permutation of 0..V-1; the backward forms its tiles from consecutive entries of this order
     * instead of consecutive vocabulary indices, so that entries with large probabilities share few
     * tiles and the filter removes the rest.  Honoured when the block-list backward runs (every
     * requested product filtered, tile_max given, no bias gradient) and col_max_key (by-product of
     * cce_b200_lse_forward_ex for the same operands) is given too; ignored otherwise.  Costs a
     * reordered copy of c in the workspace.  Both NULL: natural vocabulary order. */
    const int32_t* vocab_order;
    const int32_t* col_max_key;
    /* Optional: the staged copy of e that cce_b200_lse_forward left in its workspace for the same
     * operands (see cce_b200_lse_packed_e), with its row pitch in elements; NULL: staged here if needed. */
    const void* e_packed;
    int64_t e_packed_ld;
    /* Optional cudaEvent_t (as void*): recorded on `stream` as soon as d_e is complete.  The call then
     * computes the last dE product before the last dC product, so a caller that sums d_e across ranks
     * (vocab parallelism) can wait for this event on another stream and run the reduction while the
     * rest of dC is computed.  NULL: no event, dC before dE throughout. */
    void* de_ready_event;
    /* Optional: the cross-rank sum of dE (vocabulary parallelism) fused into the dE product.  With
     * de_peer_world > 1, de_peer_acc[r] is rank r's accumulator (cce_b200_peer_buffer_create on rank r,
     * cce_b200_peer_buffer_open here; this rank's own entry is its local pointer), each
     * [cce_b200_de_peer_rows(op.n_rows, world)][D] fp32 and all zeros.  Every rank must run the same
     * rows (same valids) with the same op.n_rows.  The product kernels then add each 128-row block of
     * this rank's partial dE into the accumulator of rank (block % world) with red.add over NVLink
     * instead of writing it locally; d_e is only cleared (rows outside valids), de_ready_event is
     * recorded after the last dE product, and the caller finishes with a barrier over the ranks,
     * cce_b200_de_peer_collect, an all-gather of the slices and cce_b200_de_peer_scatter.  At most
     * CCE_B200_MAX_PEERS ranks.  0 or 1: dE is written to d_e as described above. */
    int32_t de_peer_world;
    /* With de_ready_event: SMs the dC product launched after that event leaves free, so that the
     * caller's exchange of dE (collective kernels on another stream) can run beside it; the product
     * is a persistent kernel that otherwise holds every SM until it ends.  0: none. */
    int32_t exchange_sms;
    float* de_peer_acc[8];
} cce_b200_backward_args;
#define CCE_B200_MAX_PEERS 8

/* Gradient of sum_i d_out_i * grad_scale * (lse_i - logit_i[t_i]) + sum_i d_lse_i * lse_i
 * with respect to e, c and bias.  Accumulation is fp32 throughout.
 * Replaces cce_backward_kernel (cut_cross_entropy/cce_backward.py:346). */
size_t cce_b200_backward_workspace_bytes(const cce_b200_backward_args* a);
int cce_b200_backward(const cce_b200_backward_args* a, void* workspace, size_t workspace_bytes,
                      void* stream);

/* ---- Peer-shared buffers and the tail of the fused dE reduction (one process per GPU on one node).
 * The reference sums dE over the ranks with an all-reduce after the kernel
 * (cut_cross_entropy/vocab_parallel/utils.py:68-76, called from cce_backward.py:508-509); here the
 * product kernel adds its tiles straight into the owning rank's memory.
 *
 * create: cudaMalloc of `bytes` on the current device, cleared, with the 64-byte inter-process
 *         handle of the allocation written to handle_out (host).
 * open:   maps another process's buffer from its handle (peer access is enabled on first use).
 * close / destroy: unmap a buffer opened here / free a buffer created here. */
#define CCE_B200_PEER_HANDLE_BYTES 64
int cce_b200_peer_buffer_create(size_t bytes, void** ptr_out, void* handle_out);
int cce_b200_peer_buffer_open(const void* handle, void** ptr_out);
int cce_b200_peer_buffer_close(void* ptr);
int cce_b200_peer_buffer_destroy(void* ptr);
/* Rows of one rank's accumulator for n_rows rows over `world` ranks: whole 128-row blocks, dealt
 * round-robin. */
int64_t cce_b200_de_peer_rows(int64_t n_rows, int32_t world);
/* After a barrier over the ranks that follows every rank's cce_b200_backward: writes this rank's
 * accumulator [acc_rows][D] to slice_out in `dtype` (CCE_DT_*) and clears the accumulator.
 * status_workspace: the workspace of that cce_b200_backward call (its status word turns the slice
 * into NaN when a kernel of this rank abandoned a wait), or NULL. */
int cce_b200_de_peer_collect(float* acc, int64_t acc_rows, int64_t D, void* slice_out, int32_t dtype,
                             const void* status_workspace, void* stream);
/* cce_b200_de_peer_collect with the exchange built in: writes this rank's sums, in `dtype`, to slot
 * `rank` of every rank's gather buffer gather[r] = [world][acc_rows][D] (buffers from
 * cce_b200_peer_buffer_create / _open, 16-byte aligned; gather[rank] is this rank's own), and clears
 * the accumulator.  After a second barrier over the ranks gather[rank] holds what the all-gather of
 * the slices would have produced and goes to cce_b200_de_peer_scatter. */
int cce_b200_de_peer_collect_push(float* acc, int64_t acc_rows, int64_t D, void* const* gather, int32_t world,
                                  int32_t rank, int32_t dtype, const void* status_workspace, void* stream);
/* gathered: the ranks' slices in rank order [world][acc_rows][D]; copies row i of the reduced dE to
 * d_e[rows[i]] (rows NULL: d_e[i]); rows the list does not name are left as cce_b200_backward cleared them. */
int cce_b200_de_peer_scatter(const void* gathered, int32_t world, int64_t acc_rows, int64_t D, int32_t dtype,
                             const void* rows, int32_t rows_dtype, int64_t n_rows, const int64_t* n_rows_dev,
                             void* d_e, void* stream);

/* Synchronises `stream` and returns CCE_OK or CCE_ERR_KERNEL_WAIT; the raw word goes to *word.
 * Without this read an abandoned wait still shows: the log-sum-exp (hence the loss) and dE of that
 * call come back as NaN. */
int cce_b200_read_status(const void* workspace, void* stream, int32_t* word /* host, may be NULL */);
/* The same for the fixed scratch of cce_b200_lse_forward_static on the current device. */
int cce_b200_lse_forward_static_status(void* stream, int32_t* word /* host, may be NULL */);

const char* cce_b200_strerror(int code);
/* cudaError_t / CUresult of the most recent CCE_ERR_CUDA on this thread. */
int cce_b200_last_cuda_error(void);
int cce_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CCE_B200_H_ */
