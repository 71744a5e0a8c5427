/* C ABI of librwkv_b200.so: sm_100a kernels for the quantized ('cuda fp16i8') inference
 * path of the rwkv pip package.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *     Work is enqueued, never synchronised; the calls are safe inside stream capture
 *     (no allocation, no host synchronisation) unless stated otherwise.
 *   - Every entry point returns RWKV_OK (0) or a negative RWKV_ERR_* code and launches
 *     nothing when it returns an argument error.  The reference aborts the process with a
 *     C assert in the same situations (rwkv_pip_package/src/rwkv/cuda/wrapper.cpp:55-59,
 *     89-93, 80-82, 114-116).
 *   - "Reference" citations are paths inside the BlinkDL/ChatRWKV project;
 *     pkg/ = rwkv_pip_package/src/rwkv/.
 */
#ifndef RWKV_B200_H
#define RWKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    RWKV_OK = 0,
    RWKV_ERR_INVALID_ARG = -1,  /* bad size, NULL pointer, unknown dtype/epilogue */
    RWKV_ERR_ALIGNMENT = -2,    /* a pointer or stride breaks an alignment the kernel needs */
    RWKV_ERR_WORKSPACE = -3,    /* workspace missing or too small */
    RWKV_ERR_LAUNCH = -4,       /* the CUDA runtime rejected the launch */
    RWKV_ERR_UNSUPPORTED = -5,  /* valid request this build has no kernel for */
    RWKV_ERR_STATIC_LIMIT = -6  /* size beyond the fixed scratch of rwkv_mm8_one_static */
};

enum { RWKV_F32 = 0, RWKV_F16 = 1, RWKV_BF16 = 2 };

/* Library version (major*1000 + minor) and a static string for an error code. */
int rwkv_b200_version(void);
const char* rwkv_b200_error_string(int code);

/* ---------------------------------------------------------------------------------------
 * int8 packing — replaces the inline block pkg/model.py:818-847 (and the power-of-two
 * pre-division pkg/model.py:785-789 through `scale`).
 *
 * Logical input: fp32 W[N, M] (N = in-features = reduction index, M = out-features) read
 * as  src[j * src_stride_n + k * src_stride_m]  (strides in elements), so the loader's
 * transposed view of an [M, N] nn.Linear weight is (src_stride_n = 1, src_stride_m = N).
 * src_dtype is RWKV_F32 / RWKV_F16 / RWKV_BF16; values are widened to fp32 and multiplied
 * by `scale` (a power of two; 1.0f for no rescale) before anything else.
 * Outputs: q uint8 [N, M] with row stride q_stride (>= M); mx, rx [M] and my, ry [N] in
 * scale_dtype (RWKV_F16 or RWKV_F32); rx and ry already divided by 16 as the reference
 * stores them.  Results are bit-identical to the reference's CPU tensor ops.
 * workspace: rwkv_quantize_weight_workspace_bytes(N, M) bytes of scratch, 16-byte aligned.
 * ------------------------------------------------------------------------------------- */
size_t rwkv_quantize_weight_workspace_bytes(int64_t N, int64_t M);
int rwkv_quantize_weight(const void* src, int src_dtype, int64_t src_stride_n, int64_t src_stride_m,
                         float scale, int64_t N, int64_t M,
                         uint8_t* q, int64_t q_stride,
                         void* mx, void* rx, void* my, void* ry, int scale_dtype,
                         void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * mm8_one — replaces cuda_mm8_one<F> (pkg/cuda/operators.cu:193-246) behind
 * torch.ops.rwkv.mm8_one (pkg/cuda/wrapper.cpp:84-117).
 *
 *   y[k] += sum_j x[j] * ((w[j,k] + 0.5) * rx[k] * ry[j] + mx[k] + my[j])      k in [0, M)
 *
 * x, mx, rx, my, ry have dtype `dtype` (RWKV_F16 or RWKV_F32); y is fp32 [M] and is
 * ACCUMULATED into, as in the reference (callers pass zeros, pkg/model.py:84).  The sum is
 * evaluated in fp32 in a fixed order: two calls on equal inputs give equal bits.
 * w: uint8 [N, M], row stride w_stride >= M.  The 128-bit-load kernel is used when w is
 * 16-byte aligned, w_stride % 16 == 0 and every row has round_up(M,16) readable bytes
 * (M % 16 == 0 or w_stride >= round_up(M,16)); any other layout takes a byte-load kernel.
 * workspace: rwkv_mm8_one_workspace_bytes(N, M) bytes that were ZERO when first handed to
 * the library; each call leaves its counters zero again.  Calls sharing a workspace must
 * be ordered on one stream.
 * ------------------------------------------------------------------------------------- */
size_t rwkv_mm8_one_workspace_bytes(int64_t N, int64_t M);
int rwkv_mm8_one(int64_t N, int64_t M, const void* x, const uint8_t* w, int64_t w_stride,
                 const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                 float* y, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * mm8_one without a workspace argument — an addition of this library; the reference has no
 * counterpart (there, torch allocates whatever the operators need).
 *
 * It is meant for hosts that may not obtain device memory on behalf of the library: a
 * plugin that is handed raw tensor pointers and nothing else, a server that sizes one arena
 * at start-up and forbids later driver allocations, code running where cudaMalloc's implicit
 * device synchronisation is not acceptable.  The call allocates nothing (no cudaMalloc,
 * cudaFree or allocating library routine); the split-K scratch that rwkv_mm8_one takes as
 * `workspace` is a fixed array inside the library's device image instead.
 *
 * Same arguments, arithmetic and result as rwkv_mm8_one (y is accumulated into).  Limits and
 * rules:
 *   - M <= 32768; a larger M returns RWKV_ERR_STATIC_LIMIT and launches nothing.
 *   - The array (about 9 MiB) is held on every GPU that loads the library until the process
 *     exits, whether or not this entry point is ever called.
 *   - The first call on each device looks the array's device address up (with the caller's
 *     current device) before launching.  Make that first call outside of any stream capture,
 *     and from one thread: the per-device lookup is cached without a lock (not thread-safe).
 *   - Only the split-K kernel reads the array (matrices whose rows are not 16-byte aligned, or any
 *     matrix after rwkv_mm8_one_set_cluster(-1, 0)); the default cluster kernel for aligned matrices
 *     reduces in shared memory and leaves the array untouched.
 *   - All calls on a device share the one array, which keeps whatever the previous call left
 *     in it; the call clears the part that has to start at zero on `stream` before the kernel.
 *     Two calls that can overlap on the GPU (different streams, no dependency) race on it:
 *     order them, or use rwkv_mm8_one with separate workspaces.
 * ------------------------------------------------------------------------------------- */
int rwkv_mm8_one_static(int64_t N, int64_t M, const void* x, const uint8_t* w, int64_t w_stride,
                        const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                        float* y, void* stream);

/* ---------------------------------------------------------------------------------------
 * mm8_one with a fused epilogue, up to four matrices per launch — the building block of
 * the fused decode steps that replace att_one / ffn_one (pkg/model.py:984-992, 1034-1055)
 * and their v5/v6 forms (pkg/model.py:1007-1016, 1157-1181, 1263-1298).  `val` below is the
 * fp32 sum of mm8_one; r16() is one rounding to `dtype`, which is where the reference
 * rounds (pkg/model.py:86).
 *   RWKV_EPI_ACC_F32       y fp32:  y[k] += val
 *   RWKV_EPI_STORE         y[k] = r16(val)
 *   RWKV_EPI_SIGMOID       y[k] = sigmoid(r16(val))                     (receptance)
 *   RWKV_EPI_RELU_SQ       y[k] = relu(r16(val))^2                      (pkg/model.py:990)
 *   RWKV_EPI_RESIDUAL      y[k] = (aux[k] + r16(val)) * out_scale       (pkg/model.py:1055, 1660-1662)
 *   RWKV_EPI_MUL_RESIDUAL  y[k] = (aux[k] + aux2[k]*r16(val)) * out_scale  (pkg/model.py:991-992)
 *   RWKV_EPI_SILU          y[k] = silu(r16(val))                        (the v5/v6 gate, pkg/model.py:1170, 1284)
 *   RWKV_EPI_STORE_F32     y fp32:  y[k] = r16(val)   (the head: fp16-rounded logits returned
 *                          as fp32, pkg/model.py:1675-1677)
 * Every intermediate is rounded to `dtype` like the torch ops it replaces; out_scale is 1
 * or 0.5 (the every-6-layers halving).  y may alias aux.
 * ------------------------------------------------------------------------------------- */
enum {
    RWKV_EPI_ACC_F32 = 0,
    RWKV_EPI_STORE = 1,
    RWKV_EPI_SIGMOID = 2,
    RWKV_EPI_RELU_SQ = 3,
    RWKV_EPI_RESIDUAL = 4,
    RWKV_EPI_MUL_RESIDUAL = 5,
    RWKV_EPI_STORE_F32 = 6,
    RWKV_EPI_SILU = 7
};

/* Prologues: what the activation vector x of a problem is.
 *   RWKV_PRO_PLAIN   x[j] as given.
 *   RWKV_PRO_LN_MIX  (fp16) x is the residual stream [N]; the kernel computes
 *                    xx = layer_norm(x; ln_w, ln_b) and uses
 *                      mode 0: xx*mix + sx*(1-mix)   (pkg/model.py:986, 1036-1038)
 *                      mode 1: xx + (sx-xx)*mix      (pkg/model.py:1009-1011)
 *                      mode 2: xx                    (ln_out before the head, pkg/model.py:1668)
 *                    and stores xx to xx_out when that is not NULL.  xx_out must not alias
 *                    sx: other CTAs of the launch still read sx.
 *   RWKV_PRO_WKV4    (fp16) x is r = sigmoid(receptance); the kernel runs the RWKV-4 one-step
 *                    WKV (pkg/model.py:1044-1055) on k, v, t_decay, t_first and the state
 *                    aa, bb, pp, uses r*wkv, and stores the new state to aa_out, bb_out,
 *                    pp_out, which must not alias aa, bb, pp. */
enum { RWKV_PRO_PLAIN = 0, RWKV_PRO_LN_MIX = 1, RWKV_PRO_WKV4 = 2 };

typedef struct rwkv_mm8_problem {
    const void* x;          /* [N] activations (see the prologues) */
    const uint8_t* w;       /* [N, M] codes */
    int64_t w_stride;
    const void* mx;         /* [M] */
    const void* rx;         /* [M] */
    const void* my;         /* [N] */
    const void* ry;         /* [N] */
    void* y;                /* [M] output */
    const void* aux;        /* [M] residual input, or NULL */
    const void* aux2;       /* [M] multiplier, or NULL */
    int32_t N, M;
    int32_t epilogue;
    float out_scale;
    int32_t prologue;
    int32_t mode;
    /* RWKV_PRO_LN_MIX */
    const void* ln_w;
    const void* ln_b;
    const void* sx;
    const void* mix;
    void* xx_out;
    /* RWKV_PRO_WKV4 */
    const void* k;
    const void* v;
    const float* t_decay;
    const float* t_first;
    const float* aa;
    const float* bb;
    const float* pp;
    float* aa_out;
    float* bb_out;
    float* pp_out;
} rwkv_mm8_problem;

/* `problems` is a HOST array of 1..4 entries, read during the call. */
size_t rwkv_mm8_one_batch_workspace_bytes(const rwkv_mm8_problem* problems, int count);
int rwkv_mm8_one_batch(const rwkv_mm8_problem* problems, int count, int dtype,
                       void* workspace, size_t workspace_bytes, void* stream);
/* ---------------------------------------------------------------------------------------
 * Column-sharded decode over several GPUs (one process per GPU; no counterpart in the reference,
 * whose only multi-device feature places whole layers, pkg/model.py:684-749).  Every rank holds
 * the columns [lo, hi) of each packed matrix and a full copy of every activation buffer in a
 * region of device memory that the other ranks have mapped (rwkv_peer_*).  A launch made with
 * rwkv_mm8_one_batch_exchange stores its results into its own buffers AND into the same place of
 * every other rank's (peer_y), then publishes `signal_seq` in each rank's arrival word for this
 * rank; before touching its inputs it waits (bounded, ~0.1 s) until all `world` arrival words of
 * its own rank have reached `wait_seq` (0: no wait).  Sequence numbers grow by one per launch and
 * must be the same on every rank; `seq_base` (optional device word, same protocol on every rank)
 * is added to both on the device, so that a captured graph whose first node is rwkv_peer_advance
 * can be replayed.  RWKV_ERR_UNSUPPORTED if the launch cannot use the cluster kernel (fp16,
 * aligned rows, integer arithmetic).
 * ------------------------------------------------------------------------------------- */
#define RWKV_PEER_HANDLE_BYTES 64
typedef struct {
    void* peer_y[4][7];        /* [problem][other rank]: that rank's address of problem.y */
    uint32_t* arrived;         /* this rank's arrival words, one per rank [world] */
    uint32_t* peer_arrived[7]; /* on each other rank: the address of ITS arrival word for this rank */
    uint32_t* done_counter;    /* one zeroed word of this rank's memory (left zero) */
    uint32_t* error;           /* one word of this rank's memory; set to 1 when a wait gives up */
    const uint32_t* seq_base;  /* NULL, or a word of this rank's memory added to wait_seq and signal_seq */
    uint32_t wait_seq, signal_seq;
    int32_t world, rank;
} rwkv_mm8_exchange;
/* The same launch with flags (`exchange` may be NULL).  RWKV_MM8_WIDE_BUILD: use the kernel build that holds up
 * to 2560 rows of x per CTA (matrices with up to 20480 in-features need it) for this launch too, although it
 * would fit the ordinary build: a model with one such matrix passes it on every launch, because launches that
 * alternate between the two builds overlap worse.  No counterpart in the reference. */
#define RWKV_MM8_WIDE_BUILD 1
int rwkv_mm8_one_batch_flags(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange, int dtype,
                             int flags, void* workspace, size_t workspace_bytes, void* stream);
/* Decode launches that qualify (fp16 activations, integer arithmetic, row slices that fit its staging areas, no
 * exchange) run on a kernel that fetches its constants with bulk copies and waits for them on an mbarrier with an
 * iteration limit.  1 in *error if such a wait gave up since the last call (results were then undefined); the word
 * is cleared.  Synchronises `stream`.  RWKV_B200_LEAN=0 in the environment keeps every launch on the general kernel. */
int rwkv_mm8_one_take_error(void* stream, int* error);
/* Tuning / test hook like rwkv_mm8_one_set_variant: 0 keeps every launch on the general kernel, 1 allows the kernel
 * above, -1 lets the environment decide again.  Process-wide; not thread-safe. */
void rwkv_mm8_one_set_lean(int on);
int rwkv_mm8_one_batch_exchange(const rwkv_mm8_problem* problems, int count, const rwkv_mm8_exchange* exchange,
                                int dtype, void* workspace, size_t workspace_bytes, void* stream);
int rwkv_peer_alloc(size_t bytes, void** ptr_out);          /* zeroed device memory that can be exported */
int rwkv_peer_free(void* ptr);
int rwkv_peer_export(const void* ptr, void* handle_out);    /* RWKV_PEER_HANDLE_BYTES bytes for another process */
int rwkv_peer_open(const void* handle, void** ptr_out);     /* map another process's region (peer access over NVLink) */
int rwkv_peer_close(void* ptr);
int rwkv_peer_wait(const uint32_t* arrived, int world, uint32_t seq, const uint32_t* seq_base, uint32_t* error,
                   void* stream);
int rwkv_peer_advance(uint32_t* seq_base, uint32_t add, void* stream);   /* *seq_base += add, in stream order */

/* Tuning hooks (process-wide, not thread-safe).  split: force the number of K-splits
 * (0 = automatic).  variant: bits 0-1 force the panel width (1 = 512, 2 = 256, 3 = 128
 * columns, 0 = automatic); bit 2 switches the two-wide fp32 arithmetic off. */
void rwkv_mm8_one_set_split(int split);
void rwkv_mm8_one_set_variant(int variant);
/* How the K-splits of a column panel meet.  By default (cluster_size 0) the splits of a panel
 * are one thread-block cluster of up to 8 CTAs that adds its partial sums through distributed
 * shared memory; matrices that kernel cannot take (unaligned rows, more than 16384 in-features)
 * use global scratch and an atomic ticket.  cluster_size -1 forces the ticket kernel, 1/2/4/8
 * force a cluster size; panel_width forces the panel width in columns (0 = automatic: the narrowest
 * width with which four fifths of the resident clusters cover the launch; a negative value plans for
 * that many clusters).  Forcing
 * a split or a width with the two hooks above also selects the ticket kernel.  No counterpart in
 * the reference. */
void rwkv_mm8_one_set_cluster(int cluster_size, int panel_width);
/* Tuning: launches whose matrices have `total_columns` output columns in all are planned for `clusters`
 * clusters (0 = back to automatic).  Up to 16 entries, process-wide. */
void rwkv_mm8_one_set_plan(int64_t total_columns, int clusters);


/* ---------------------------------------------------------------------------------------
 * mm8 stream — one decode step (the same list of dependent mm8_one problems with fused prologues
 * and epilogues that rwkv_mm8_one_batch takes launch by launch) as ONE persistent cooperative
 * kernel, one CTA per SM, over a re-tiled copy of the codes.  Replaces the per-token loop of
 * RWKV.forward over att_one / ffn_one (pkg/model.py:1477-1677) for T = 1; no counterpart in the
 * reference.  fp16 only; every N a multiple of 8; x, ry, my and the prologue vectors 16-byte
 * aligned.
 *
 * Layout ("weight stream"): the output columns of every matrix are dealt to the CTAs in units of
 * four, so a CTA owns whole dot products (no split-K, no reduction between CTAs).  The bytes a CTA
 * needs for the whole step are one contiguous region of the stream, in the order its threads
 * consume them: 8-byte cells of 2 rows x 4 columns, row-interleaved for dp2a.  A producer warp
 * moves the region through a ring of 16 KB shared-memory slots with bulk asynchronous copies and
 * runs ahead of the arithmetic across matrix and phase boundaries.  Between phases the CTAs meet
 * at a grid barrier (every wait is bounded: after 2 s it sets the error word and carries on).
 * Arithmetic: x * ry as 30-bit (optionally 24- or 16-bit) fixed point, exact integer sums (see
 * csrc/mm8_stream.cu).
 *
 *   rwkv_mm8_stream_ctas()          CTAs of the grid on the current device (its SM count).
 *   rwkv_mm8_stream_weight_bytes()  size of the weight stream for `problems` (all phases' problems
 *                                   back to back; only w, w_stride, N, M are read).
 *   rwkv_mm8_stream_pack()          re-tiles the codes into `wstream` (device, 16-byte aligned).
 *   rwkv_mm8_stream_table_bytes()   size of the phase table.
 *   rwkv_mm8_stream_plan()          HOST-side: writes the table for the same problems, counts[p] =
 *                                   problems of phase p (1..4), into `table_host`.  Copy it to the
 *                                   device; keep the host copy for rwkv_mm8_stream_run.
 *                                   RWKV_ERR_UNSUPPORTED when a problem does not meet the limits.
 *   rwkv_mm8_stream_run()           enqueues one step.  sync_words: two device words (barrier
 *                                   counter, error); the call clears the counter in stream order.
 *                                   trace: NULL, or n_phases x 2 x 16 uint64 (device) receiving
 *                                   %globaltimer stamps of CTAs 0 and 1 per phase: barrier
 *                                   arrival, barrier passed, prologue done, matrices done,
 *                                   LayerNorm statistics done, activations computed, their
 *                                   maxima reduced, -; then for the phase's first matrix: start,
 *                                   first stage in shared memory, last stage multiplied, the two
 *                                   barriers of the column reduction.
 *   rwkv_mm8_stream_take_error()    synchronises `stream`, returns and clears the error word.
 * ------------------------------------------------------------------------------------- */
int rwkv_mm8_stream_ctas(void);
/* Tuning hook (process-wide, not thread-safe): digit planes of x * ry the matrices are multiplied with in
 * tables planned from now on: 4 (default) = 30-bit fixed point, 3 = 24-bit (error per product at most
 * 2^-24 of the largest |x * ry|, the mantissa of an fp32 product), 2 = 16-bit.  The kernel's speed did not
 * depend on it when measured (it is bound by the per-phase work, not by the dot products). */
void rwkv_mm8_stream_set_planes(int planes);
size_t rwkv_mm8_stream_weight_bytes(const rwkv_mm8_problem* problems, int n_problems, int n_ctas);
int rwkv_mm8_stream_pack(const rwkv_mm8_problem* problems, int n_problems, int n_ctas, void* wstream,
                         size_t wstream_bytes, void* stream);
size_t rwkv_mm8_stream_table_bytes(int n_phases);
int rwkv_mm8_stream_plan(const rwkv_mm8_problem* problems, const int32_t* counts, int n_phases, int dtype,
                         int n_ctas, void* table_host, size_t table_bytes);
int rwkv_mm8_stream_run(const void* table_device, const void* table_host, const void* wstream,
                        uint32_t* sync_words, uint64_t* trace, void* stream);
int rwkv_mm8_stream_take_error(uint32_t* sync_words, void* stream, int* error_out);

/* ---------------------------------------------------------------------------------------
 * mm8_seq — replaces cuda_mm8_seq<F> (pkg/cuda/operators.cu:102-154) behind
 * torch.ops.rwkv.mm8_seq (pkg/cuda/wrapper.cpp:50-83).
 *
 *   y[i,k] = sum_j x[i,j] * ((w[j,k] + 0.5) * rx[k] * ry[j] + mx[k] + my[j])   i in [0, B)
 *
 * x [B, N] row stride x_stride, y [B, M] row stride y_stride, both in `dtype`, fp32
 * accumulation, one rounding to `dtype` at the store (operators.cu:138).
 * Two kernels: from 8 rows up, fp16 operands whose w is 8-byte aligned (pointer, stride, M)
 * run on the tensor cores (tcgen05 UMMA, fp32 accumulation in tensor memory; x*ry enters as
 * an exact hi + lo pair of fp16 values) and need `workspace` =
 * rwkv_mm8_seq_workspace_bytes(B, N, M) bytes, 256-byte aligned, zero when first handed over;
 * everything else (or workspace == NULL) runs on a CUDA-core kernel that accepts any layout.
 * rwkv_mm8_seq_set_path: 0 automatic, 1 CUDA cores only, 2 tensor cores whenever possible; adding 4
 * makes the tensor-core kernel multiply fp16(x*ry) in ONE pass instead of the exact hi + lo pair
 * (about 1e-4 of the output's RMS less accurate, 10-35 % faster at T = 1024; off by default); adding 8
 * keeps one CTA per output tile (by default launches with an even number of 128-row tiles and no K
 * split run as clusters of two CTAs sharing one 256-row UMMA, tcgen05 cta_group::2; same results).
 * rwkv_mm8_seq_tc_take_error synchronises `stream` and returns/clears the workspace's error
 * word (1 if a bounded wait inside the tensor-core kernel gave up; outputs then undefined).
 * ------------------------------------------------------------------------------------- */
void rwkv_mm8_seq_set_path(int path);
int rwkv_mm8_seq_tc_take_error(void* workspace, void* stream, int* error_out);
size_t rwkv_mm8_seq_workspace_bytes(int64_t B, int64_t N, int64_t M);
/* mm8_seq with a fused epilogue: RWKV_EPI_STORE, _SIGMOID, _RELU_SQ, _RESIDUAL (aux), _MUL_RESIDUAL (aux, aux2)
 * or _SILU applied to the fp32 sums with the roundings listed for rwkv_mm8_one_batch; aux, aux2: [B, M] in
 * `dtype`, rows aux_stride / aux2_stride elements apart; y may alias aux.  What ffn_seq / cuda_att_seq apply
 * between matmuls (pkg/model.py:995-1004, 1346-1360). */
int rwkv_mm8_seq_epi(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                     const uint8_t* w, int64_t w_stride,
                     const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                     void* y, int64_t y_stride, int epilogue, const void* aux, int64_t aux_stride,
                     const void* aux2, int64_t aux2_stride, float out_scale,
                     void* workspace, size_t workspace_bytes, void* stream);
int rwkv_mm8_seq(int64_t B, int64_t N, int64_t M, const void* x, int64_t x_stride,
                 const uint8_t* w, int64_t w_stride,
                 const void* mx, const void* rx, const void* my, const void* ry, int dtype,
                 void* y, int64_t y_stride, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * WKV-v4 — replaces cuda_wkv_forward<F> (pkg/cuda/operators.cu:11-58) behind
 * torch.ops.rwkv.wkv_forward (pkg/cuda/wrapper.cpp:27-48).
 * w = -exp(time_decay), u = time_first: fp32 [C].  k, v, y: [B, T, C] in kv_dtype
 * (RWKV_F16 or RWKV_F32).  aa, bb, pp: fp32 [B, C] state, updated in place.
 * rwkv_wkv4_seq is the same with two additions.  `workspace` (rwkv_wkv4_workspace_bytes, 16-byte aligned;
 * may be NULL) lets sequences of more than 32 steps run parallel in time: chunks of 32 steps are
 * summarised from the empty state, every chunk folds the summaries before it into the caller's state
 * and then runs its own steps (results equal the sequential recurrence up to fp32 rounding of that
 * fold).  Without it the steps run one after the other, as rwkv_wkv4_forward does.  `r` (may be NULL;
 * [B, T, C] in kv_dtype): y = r * wkv with the roundings of cuda_att_seq (pkg/model.py:1359-1360).
 * ------------------------------------------------------------------------------------- */
size_t rwkv_wkv4_workspace_bytes(int64_t B, int64_t T, int64_t C);
int rwkv_wkv4_seq(int64_t B, int64_t T, int64_t C, const float* w, const float* u,
                  const void* k, const void* v, const void* r, void* y, int kv_dtype,
                  float* aa, float* bb, float* pp, void* workspace, size_t workspace_bytes, void* stream);
int rwkv_wkv4_forward(int64_t B, int64_t T, int64_t C, const float* w, const float* u,
                      const void* k, const void* v, void* y, int kv_dtype,
                      float* aa, float* bb, float* pp, void* stream);

/* ---------------------------------------------------------------------------------------
 * WKV5 / WKV6 for the model's sequence path, and the pointwise pieces around them — replace what
 * cuda_att_seq_v5_2 / cuda_att_seq_v6_0 do in torch between the matmuls (pkg/model.py:1379-1439).
 *
 * rwkv_wkv56_seq: the recurrence of rwkv_wkv5_forward (per_token_w = 0, w [H*N]) or rwkv_wkv6_forward
 * (per_token_w = 1, w [T, C]) with r, k, v in in_dtype and u, y in out_dtype (the operators' three
 * uniform dtypes, or fp16 in / fp32 out: the model's fp16-rounded r, k, v without a widened copy,
 * pkg/model.py:1413, 1425-1427).  model_layout = 1: `state` is [H, key, value], the transpose the model
 * keeps in its state list (pkg/model.py:1376, 1384).  The new state goes to state_out (may be `state`:
 * in place; a separate buffer leaves the caller's state untouched, as the reference's copy does).  With `workspace`
 * (rwkv_wkv56_workspace_bytes, 16-byte aligned; NULL allowed) sequences of more than 64 steps run
 * parallel in time: chunk sums from an empty state, a scan of the chunk-start states, the chunks again
 * for y (results equal the sequential recurrence up to fp32 rounding).
 * rwkv_v6_seq_mix: the five token-shift mixes from xx [T, D] (LayerNorm output), the previous token's
 * xx (`state` [D]; with state_stride != 0 every row is its own sequence with its state at state + t *
 * state_stride: batched decode), the low-rank offsets m [5, T, D] and time_maa_{w,k,v,r,g}; out5: five [T, D].
 * rwkv_tanh_regroup_f16: out[g, t, r] = tanh(in[t, g, r]) (G = 1: plain tanh, in place allowed).  rwkv_v6_seq_decay: out[T, D] = exp(-exp(time_decay + float(d2))) in fp32.
 * rwkv_v56_seq_gn_gate: group-norm of y [T, H*N] over each head's N channels (eps), ln_x weight / bias in
 * fp32, rounded to fp16 and multiplied with the gate g [T, H*N] in fp16.
 * ------------------------------------------------------------------------------------- */
size_t rwkv_wkv56_workspace_bytes(int64_t T, int64_t C, int64_t H);
int rwkv_wkv56_seq(int per_token_w, int64_t T, int64_t C, int64_t H, const float* state, float* state_out, int model_layout,
                   const void* r, const void* k, const void* v, const float* w, const void* u, void* y,
                   int in_dtype, int out_dtype, void* workspace, size_t workspace_bytes, void* stream);
int rwkv_v6_seq_mix(int64_t T, int64_t D, const void* xx, int64_t xx_stride, const void* state, int64_t state_stride,
                    const void* m, const void* const* maa5, void* const* out5, void* stream);
int rwkv_tanh_regroup_f16(int64_t T, int64_t G, int64_t R, const void* in, void* out, void* stream);
int rwkv_v6_seq_decay(int64_t T, int64_t D, const float* time_decay, const void* d2, float* out, void* stream);
int rwkv_v56_seq_gn_gate(int64_t T, int64_t H, int64_t N, const float* y, const float* ln_w, const float* ln_b,
                         const void* g, void* out, float eps, void* stream);

/* ---------------------------------------------------------------------------------------
 * WKV5 / WKV6 — replace cuda_forward_{bf16,fp16,fp32} of pkg/cuda/rwkv5.cu:8-88 and
 * pkg/cuda/rwkv6.cu:8-87 behind rwkv5.forward_* / rwkv6.forward_*
 * (pkg/cuda/rwkv5_op.cpp:12-34, pkg/cuda/rwkv6_op.cpp:12-34).
 * state fp32 [H, N, N] in the kernel layout [head, value index, key index], updated in
 * place (B must be 1, as in the reference).  r, k, v, y: [T, C] in `dtype`; u: [H*N] in
 * `dtype`.  v5: w fp32 [H*N] = exp(-exp(decay)).  v6: w fp32 [T, C], already
 * exp(-exp(.)) (pkg/model.py:959).  The head size N = C / H may be 16, 32, 64 or 128 and
 * is a run-time argument here (the reference compiles it in with -D_N_).
 * ------------------------------------------------------------------------------------- */
int rwkv_wkv5_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                      const void* r, const void* k, const void* v, const float* w, const void* u,
                      void* y, int dtype, void* stream);
int rwkv_wkv6_forward(int64_t B, int64_t T, int64_t C, int64_t H, float* state,
                      const void* r, const void* k, const void* v, const float* w, const void* u,
                      void* y, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * LayerNorm + token-shift mixes in one launch — the opening lines of att_one / att_seq /
 * ffn_one / ffn_seq (pkg/model.py:985-987, 996-999, 1035-1038, 1059-1063) and of their
 * RWKV-6 forms (pkg/model.py:1008-1011, 1020-1024).  fp16 only.
 *   xx[t]  = layer_norm(x[t]; ln_w, ln_b)                 (fp32 statistics, eps 1e-5)
 *   prev   = t == 0 ? sx : xx[t-1]
 *   mode 0: out_m[t] = xx[t]*mix_m + prev*(1 - mix_m)
 *   mode 1: out_m[t] = xx[t] + (prev - xx[t])*mix_m
 * with one fp16 rounding per torch op of the reference.  mix_m is [D] (mix_stride 0) or
 * [T, D].  `mix` and `out` are HOST arrays of n_mix (0..5) device pointers.  xx_out
 * (optional) receives xx; new_state (optional, may alias sx only when T == 1) receives
 * xx[T-1].
 * ------------------------------------------------------------------------------------- */
int rwkv_ln_mix(int64_t T, int64_t D, const void* x, int64_t x_stride, const void* sx,
                const void* ln_w, const void* ln_b, int mode, int n_mix,
                const void* const* mix, int64_t mix_stride, void* const* out, int64_t out_stride,
                void* xx_out, int64_t xx_stride, void* new_state, void* stream);
/* The same for rows that are independent sequences (batched decode, one token each; no counterpart in the
 * reference, which has no batch dimension): prev of row t = sx + t * sx_stride (sx_stride != 0; 0 = rwkv_ln_mix);
 * take the new per-sequence states from xx_out. */
int rwkv_ln_mix_rows(int64_t T, int64_t D, const void* x, int64_t x_stride, const void* sx, int64_t sx_stride,
                     const void* ln_w, const void* ln_b, int mode, int n_mix,
                     const void* const* mix, int64_t mix_stride, void* const* out, int64_t out_stride,
                     void* xx_out, int64_t xx_stride, void* new_state, void* stream);

/* ---------------------------------------------------------------------------------------
 * rwkv_embed_row: out[0..D) = emb[*token] (fp16; `token` a device int64), the embedding lookup that opens a
 * decode step (pkg/model.py:1475 `x = w['emb.weight'][tokens[0]]`) as a kernel of this library, so that the
 * launch after it starts under it.  An id outside [0, V) reads the nearest valid row.
 * ------------------------------------------------------------------------------------- */
int rwkv_embed_row(int64_t D, int64_t V, const void* emb, int64_t row_stride, const int64_t* token, void* out,
                   void* stream);

/* ---------------------------------------------------------------------------------------
 * RWKV-4 one-step WKV — the fp32 island of att_one (pkg/model.py:1044-1055).
 * r (after sigmoid), k, v: fp16 [C]; t_decay = -exp(time_decay), t_first: fp32 [C];
 * aa, bb, pp: fp32 [C] updated in place; out = r * wkv in fp16 (the operand of the output
 * matmul).
 * ------------------------------------------------------------------------------------- */
int rwkv_wkv4_one(int64_t C, const float* t_decay, const float* t_first, const void* r,
                  const void* k, const void* v, float* aa, float* bb, float* pp, void* out,
                  void* stream);

/* ---------------------------------------------------------------------------------------
 * One-token pieces of att_one_v5_1 / att_one_v6_0 that are not packed matmuls (fp16
 * activations; pkg/model.py:1157-1181, 1263-1298).  They allocate nothing.
 *
 * rwkv_v6_token_shift (model.py:1264-1276):
 *   xx = layer_norm(x; ln_w, ln_b);  dd = state - xx;  new_state <- xx   (new_state may alias state)
 *   m[0..4] = tanh((xx + dd*maa_x) @ tm_w1 [D, 5*Lm]) viewed [5, Lm], times tm_w2 [5, Lm, D]
 *   out5[f] = xx + dd * (maa5[f] + m[f])        f = w, k, v, r, g
 * xx_out and d_out receive xx and dd.  maa5 / out5: HOST arrays of five device pointers.
 * scratch: rwkv_v6_scratch_bytes(D, 5*Lm) bytes (D, Ld for the decay).  D % 8 == 0, D <= 8192.
 *
 * rwkv_v6_decay (model.py:1286-1287):
 *   w_out = exp(-exp(time_decay + tanh(wx @ td_w1 [D, Ld]) @ td_w2 [Ld, D]))      fp32 [D]
 *
 * rwkv_wkv56_one (model.py:1174-1179, 1289-1294): for each head, with fp16-rounded r, k, v,
 *   out_i = sum_j r_j (u_j k_j v_i + S[j][i]);  S'[j][i] = w_j S[j][i] + k_j v_i
 * with S = state and S' = new_state (may alias) in the model's layout [H, N(key), N(value)], then group_norm over each head
 * (eps 64e-5, fp32 lnx_w / lnx_b), cast to fp16 and times the gate g.  w, u: fp32 [H*N]
 * (RWKV-5.2: exp(-exp(time_decay)); RWKV-6: rwkv_v6_decay's output).  N <= 256.
 *
 * rwkv_v6_att_pre: rwkv_v6_token_shift followed by rwkv_v6_decay (of out5[0] = wx) as ONE launch
 * of a single 8-CTA cluster that exchanges the low-rank intermediates through distributed shared
 * memory; same values, no scratch.  Returns RWKV_ERR_UNSUPPORTED (and launches nothing) unless
 * 5*Lm and Ld are multiples of 8 and D <= 8192: callers then use the two calls above.
 * With td_w1, td_w2, time_decay and w_out all NULL it does the token shift alone (a caller can then
 * run rwkv_v6_decay on another stream beside the matmuls that only need the shifted vectors).
 * ------------------------------------------------------------------------------------- */
size_t rwkv_v6_scratch_bytes(int64_t D, int64_t rank);
int rwkv_v6_att_pre(int64_t D, int64_t Lm, int64_t Ld, const void* x, const void* state, void* new_state,
                    const void* ln_w, const void* ln_b, const void* maa_x, const void* const* maa5,
                    const void* tm_w1, const void* tm_w2, const void* td_w1, const void* td_w2,
                    const float* time_decay, void* xx_out, void* d_out, void* const* out5, float* w_out,
                    void* stream);
int rwkv_v6_token_shift(int64_t D, int64_t Lm, const void* x, const void* state, void* new_state,
                        const void* ln_w, const void* ln_b,
                        const void* maa_x, const void* const* maa5, const void* tm_w1, const void* tm_w2,
                        float* scratch, size_t scratch_bytes, void* xx_out, void* d_out, void* const* out5,
                        void* stream);
int rwkv_v6_decay(int64_t D, int64_t Ld, const void* wx, const void* td_w1, const void* td_w2,
                  const float* time_decay, float* scratch, size_t scratch_bytes, float* w_out, void* stream);
int rwkv_wkv56_one(int64_t H, int64_t N, const void* r, const void* k, const void* v, const float* w,
                   const float* u, const float* state, float* new_state, const float* lnx_w,
                   const float* lnx_b, const void* g, void* out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Token sampling on the device — PIPELINE.sample_logits and the penalty bookkeeping of
 * PIPELINE.generate (pkg/utils.py:55-135), without the host round trip and without a sort.
 *
 * logits: fp32 [V] as forward() returns them (not modified), V <= 65536.  In order: banned[id] != 0 sets a logit to
 * -inf; every id with seen[id] != 0 loses alpha_presence + occurrence[id] * alpha_frequency (utils.py:97-100);
 * softmax; temperature == 0 means temperature 1 and top_p 0 (greedy); probabilities below the nucleus cutoff are
 * dropped (the cutoff is the largest probability v whose probabilities >= v sum to at least top_p; if nothing
 * reaches top_p only the most likely token stays, as in the reference); all but the top_k most likely are dropped
 * (0 = off; ties by lowest id); p ** (1 / temperature); one draw by inverse CDF in id order on
 * uniforms[*counter % n_uniforms] (numbers in [0, 1) supplied by the caller; NULL = 0.5; 0 picks the lowest id that
 * has mass), after which *counter grows by one.  *token_out receives the id.  probs_out (or NULL) receives the
 * normalised distribution the draw was made from.  Then, when occurrence / seen are given (both or neither):
 * occurrence[id] *= alpha_decay for every seen id, occurrence[token] += token_weight[token] (NULL = 1), seen[token]
 * = 1 (utils.py:111-122).  One cluster of 8 CTAs; safe inside stream capture.
 * ------------------------------------------------------------------------------------- */
int rwkv_sample_logits(int64_t V, const float* logits, float temperature, float top_p, int64_t top_k,
                       float* occurrence, unsigned char* seen, const unsigned char* banned, const float* token_weight,
                       float alpha_presence, float alpha_frequency, float alpha_decay,
                       const float* uniforms, int64_t n_uniforms, uint32_t* counter,
                       int64_t* token_out, float* probs_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RWKV_B200_H */
