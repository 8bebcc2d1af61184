/* det_b200 — C ABI of the B200 (sm_100a) backend for det.
 *
 * Part 1 is the drop-in boundary: the same symbols, argument order, struct layouts and error behaviour that det's
 * FFI crate binds (crates/det-sys/src/lib.rs:54-228, declared in C by kernels/cuda/det_cuda.h), so that
 * crates/det/src/cuda.rs can drive this library unchanged.  Part 2 holds additive entry points that the reference does
 * not have (weight repack for the streaming GEMV, graph replay of the decode step, device-side token feedback).
 *
 * Conventions (kernels/cuda/det_cuda.h:1-5): every data pointer is a DEVICE pointer obtained from det_malloc unless a
 * parameter says "host"; tensors are row-major fp32 unless noted; work is issued in program order on one in-order
 * queue.  A stream argument of 0 selects that queue (det_cuda_stream()).  Failures of the CUDA runtime and malformed
 * shapes print to stderr and abort(), as the reference does (kernels/cuda/common.cuh:8-9); det_init and det_malloc
 * report through their return values.
 */
#ifndef DET_B200_H
#define DET_B200_H
#include <stddef.h>
#include <stdint.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ================================================================================================================
 * Part 1 — reference-compatible symbols
 * ============================================================================================================== */

/* ---- runtime (replaces kernels/cuda/runtime.cu:83-121; bound at crates/det-sys/src/lib.rs:56-69) */
int det_init(void);                      /* 0 on success; selects the current device                               */
const char* det_device_name(void);
void* det_malloc(size_t bytes);          /* zero-filled device buffer, NULL when the allocation fails              */
void det_free(void* p);                  /* waits for pending work before releasing                                */
size_t det_allocated_bytes(void);
void det_sync(void);                     /* waits for everything issued so far; aborts on a kernel error           */
void det_flush(void);                    /* nothing to do: launches are submitted eagerly                          */
void det_memset(void* p, int value, size_t bytes, cudaStream_t st);
void det_memcpy(void* dst, const void* src, size_t bytes, cudaStream_t st);   /* any direction                     */
void* det_cuda_stream(void);             /* the queue det's work runs on                                           */

/* ---- a quantized linear y = W x, W[N][K] (kernels/cuda/det_cuda.h:26-32, docs/SPEC.md §2)
 * bits in {4, 6, 8}: wq is the reference layout, row-major packed codes [N][K/32 * bytes_per_32].
 * bits | DET_LAYOUT_STREAM: wq points at a buffer produced by det_linear_repack (Part 2).                          */
typedef struct {
    const uint8_t* wq;
    const float* c;      /* [N]        */
    const uint16_t* m;   /* [N][K/128] */
    int N, K, bits;
} det_qlinear;

/* ---- glue (replaces kernels/cuda/norm.cu:126-227; det_cuda.h:34-43)
 * Quantization is quant_act_i8g (spec/quant.rs:21-49): sx[M] and, when mx != NULL, mx[M][n/128]; mx == NULL selects
 * the per-row form quant_act_i8 (spec/quant.rs:7-16).                                                               */
void det_rmsnorm_quant(const float* x, const float* w, float eps, int M, int n, float* y /* may be NULL */,
                       int8_t* xq /* may be NULL */, float* sx, uint16_t* mx, cudaStream_t st);
void det_quant(const float* x, int M, int n, int8_t* xq, float* sx, uint16_t* mx, cudaStream_t st);
void det_embed(const uint16_t* table_bf16, const int* ids, int M, int H, float* x, cudaStream_t st);
void det_add(float* x, const float* y, long long n, cudaStream_t st);                       /* x += y             */
void det_silu_mul_quant(const float* g, const float* u, int M, int n, float* h /* may be NULL */, int8_t* hq,
                        float* sh, uint16_t* mh, cudaStream_t st);
void det_argmax(const float* logits, int M, int V, int* out, cudaStream_t st);              /* lowest index wins  */

/* ---- integer GEMM (replaces kernels/cuda/gemm.cu:1030-1061; det_cuda.h:45-57; docs/SPEC.md §3)
 *   acc[t][n] = sum_g (m[n][g] * mx[t][g]) * sum_{k in g} wq[n][k] * xq[t][k]      exact, int64
 *   y[t][n]   = ((float)acc * c[n]) * sx[t]
 * accumulate != 0: y += result (one fp32 add).  nparts > 1: column range [offs[i], offs[i+1]) (the last one ends at N)
 * goes to dsts[i], a [M][width_i] buffer; offs and dsts are HOST arrays read before the call returns.               */
void det_gemm(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
              cudaStream_t st);
void det_gemm_ex(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
                 int accumulate, int nparts, const int* offs, float* const* dsts, cudaStream_t st);
/* Two linears over the same input rows as one launch (both in the det_linear_expand layout with the same K: otherwise
 * two det_gemm_ex calls): the row tiles of L2 follow those of L1 in the grid.  Outputs as det_gemm_ex's nparts / offs /
 * dsts form (nparts >= 1).  A small linear beside a wide one — the Gated DeltaNet a|b projection beside qkv|z — otherwise
 * pays a launch of its own.  Same values as the two separate calls.                                                   */
void det_gemm_pair(const det_qlinear* L1, const det_qlinear* L2, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                   int nparts1, const int* offs1, float* const* dsts1, int nparts2, const int* offs2, float* const* dsts2,
                   cudaStream_t st);
/* Scratch protocol of the reference's large-M path (det_cuda.h:52-57).  Kept so that callers that follow it link and
 * run: this backend's kernels need no such scratch, so the registration is accepted and ignored.                    */
size_t det_gemm_scratch_bytes(int M, int K);
void det_gemm_set_scratch(void* p, size_t bytes);

/* ---- gated attention (replaces kernels/cuda/attn.cu:856-930; det_cuda.h:59-83; docs/SPEC.md §5.1)
 * Cache: kq[pos][n_kv][hd] int8, sk[pos][n_kv] fp32, vq[pos][n_kv][hd] int16.                                       */
typedef struct {
    const float* q_norm;        /* [hd] */
    const float* k_norm;        /* [hd] */
    const float* v_scale;       /* [n_kv] */
    const float* v_inv_scale;   /* [n_kv] */
} det_attn_layer;
typedef struct {
    int8_t* kq;
    float* sk;
    int16_t* vq;
    int capacity;
    int8_t* vlo;   /* unused (Metal keeps V as two planes) */
    int8_t* vhi;
} det_kv_cache;
/* M new tokens at positions pos0 .. pos0+M-1: qg[M][n_h*2*hd] (per head q | gate), k[M][n_kv*hd], v[M][n_kv*hd],
 * rope tables [pos][rot/2].  Writes the cache rows, attends each token to positions <= its own, applies
 * sigmoid(gate), writes o[M][n_h*hd].  scratch >= det_attn_scratch_bytes(M, n_h, hd).                              */
void det_attention(const det_attn_layer* L, const det_kv_cache* kv, const float* qg, const float* k, const float* v,
                   const float* rope_cos, const float* rope_sin, int rot, float eps, int M, int pos0, int n_h,
                   int n_kv, int hd, float* o, void* scratch, cudaStream_t st);
size_t det_attn_scratch_bytes(int M, int n_h, int hd);
/* Same, with pos0 read from device memory at execution time so the launch can be replayed from a graph; sized for
 * any pos0 <= max_pos (det_cuda.h:77-83).                                                                            */
void det_attention_dev(const det_attn_layer* L, const det_kv_cache* kv, const float* qg, const float* k,
                       const float* v, const float* rope_cos, const float* rope_sin, int rot, float eps, int M,
                       const int* pos0_dev, int max_pos, int n_h, int n_kv, int hd, float* o, void* scratch,
                       cudaStream_t st);

/* ---- Gated DeltaNet (replaces kernels/cuda/gdn.cu:271-309; det_cuda.h:85-105; docs/SPEC.md §5.2) */
typedef struct {
    const float* conv;      /* [conv_dim][4], oldest tap first */
    const float* A;         /* [n_v] */
    const float* dt_bias;   /* [n_v] */
    const float* norm;      /* [dv]  */
} det_gdn_layer;
typedef struct {
    float* conv_state;      /* [3][conv_dim], oldest first */
    float* S;               /* [n_v][dk][dv] */
} det_gdn_state;
/* qkv[M][conv_dim], conv_dim = 2*n_k*dk + n_v*dv; z[M][n_v*dv]; a[M][n_v]; b[M][n_v] -> on[M][n_v*dv].
 * det_gdn_ex also exports gin[M][n_k][2*dk + rep*dv + 2*rep] (q | k | v[rep] | beta[rep] | decay[rep]) and
 * gout[M][n_v][dv] (mixer output before the gated norm); either may be NULL.                                        */
void det_gdn(const det_gdn_layer* L, det_gdn_state* S, const float* qkv, const float* z, const float* a,
             const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
             cudaStream_t st);
size_t det_gdn_scratch_bytes(int M, int n_k, int n_v, int dk, int dv);
void det_gdn_ex(const det_gdn_layer* L, det_gdn_state* S, const float* qkv, const float* z, const float* a,
                const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
                float* gin, float* gout, cudaStream_t st);

/* ---- deterministic sampling (replaces kernels/cuda/sample.cu:237-287; det_cuda.h:107-112; docs/SPEC.md §5.5)
 * z[M]: raw 64-bit draws (splitmix64, advanced by the host).                                                        */
void det_sample(const float* logits, int M, int V, float inv_temp, const unsigned long long* z, int* out,
                cudaStream_t st);
void det_sample_topkp(const float* logits, int M, int V, float inv_temp, int top_k, float top_p,
                      const unsigned long long* z, int* out, void* scratch, cudaStream_t st);
size_t det_sample_scratch_bytes(int M, int V);

/* ---- primitive test hook (replaces kernels/cuda/runtime.cu:40-77,123-127; det_cuda.h:114-118)
 * op: 0 exp_f, 1 log_f, 2 softplus_f, 3 sigmoid_f, 4 silu_f, 5 int64 (bits of x[2i], x[2i+1]) -> fp32 into out[2i],
 *     6 rint, 7 1/x, 8 sqrt, 9 x*y, 10 x+y (y = x reversed), 11 treesum of each of M rows of n (n <= 8192) -> out[M],
 *     12 same as 5 through the plain cast, 13 rint to int32 (saturating) back to fp32, 14 x/y, 15 x-y, 16 max(x,y).  */
void det_test_prim(int op, const float* x, int M, int n, float* out, cudaStream_t st);

/* ================================================================================================================
 * Part 2 — additions (no counterpart in the reference unless noted)
 * ============================================================================================================== */

/* Layout tag OR-ed into det_qlinear.bits once wq points at a det_linear_repack buffer. */
#define DET_LAYOUT_STREAM 0x100
/* ... whose rows are interleaved: a linear of two equal halves (gate | up), physical row 2i = row i of the first half,
 * row 2i+1 = row i of the second (det_linear_repack_pairs).  Outputs are still delivered in the linear's own order.  */
#define DET_LAYOUT_PAIRS 0x400

/* Streaming layout for the decode GEMV.  The reference's Rust glue builds its device layout in Backend::linear
 * (crates/det/src/cuda.rs:139-163: row-major codes, c and m split out); Metal and x86 repack there
 * (metal.rs:95-122, x86/gemm.rs:59-134).  This is that hook for B200: `src` describes device arrays in the reference
 * layout; `dst` receives det_linear_repack_bytes(N, K, bits) bytes in which four output rows x one 1024-wide chunk of K
 * form one contiguous 16-byte-aligned record [codes of the 4 rows, regrouped for 128-bit shared-memory loads |
 * m[4][8]]; a record is one bulk copy.  c and m of `src` stay in use (c is read from its own array), so the
 * det_qlinear that names the repacked buffer keeps src's c and m pointers.                                         */
size_t det_linear_repack_bytes(int N, int K, int bits);
void det_linear_repack(const det_qlinear* src, void* dst, cudaStream_t st);
void det_linear_repack_pairs(const det_qlinear* src, void* dst, cudaStream_t st);   /* N even; tag with DET_LAYOUT_PAIRS */

/* Tensor-core layout for prefill (M > 8): signed int8 codes in tile-major order [ceil(N/128)][K/128][128 rows][128 codes]
 * (each 16 KB box a TMA load fetches is contiguous; det_linear_expand_bytes(N, K) bytes, the last row tile zero padded),
 * tagged bits | DET_LAYOUT_INT8 in det_qlinear.  det_gemm_ex then runs the tcgen05 kind::i8 kernel.  Like the repack
 * above this belongs in Backend::linear (crates/det/src/cuda.rs:139-163).                                            */
#define DET_LAYOUT_INT8 0x200
size_t det_linear_expand_bytes(int N, int K);
void det_linear_expand(const det_qlinear* src, void* dst, cudaStream_t st);

/* Decode GEMV with its neighbours fused in (M <= 8 rows, streaming layout; no reference counterpart as one call).  The
 * reference runs a decode sub-block as separate kernels — det_rmsnorm_quant / det_quant, det_gemm_ex per linear,
 * det_silu_mul_quant (crates/det/src/qwen35.rs:33-36, 73-74, 121-143); here one launch can carry
 *   - src != NULL: the activation quantization as the GEMV's prologue.  Every CTA rebuilds the quantized row from the
 *     fp32 input while its weight ring fills: kind DET_ACT_RMSNORM (a = x[M][K], b = norm weight [K], eps) or
 *     DET_ACT_PLAIN (a = x[M][K]).  xq / sx / mx of src, when given, receive the row as det_rmsnorm_quant / det_quant
 *     would have written it (stored by one CTA, for other consumers).  src == NULL: xq, sx, mx are the input rows.
 *   - lin2 != NULL: a second, small W8 streaming-layout linear over the same rows (the GDN a|b projection beside
 *     qkv|z), with its own outputs (y2 / nparts2 / offs2 / dsts2).
 *   - h != NULL (lin in the pairs layout): h[M][N/2] = silu_f(gate) * up, the product det_silu_mul_quant forms before it
 *     quantizes, instead of the outputs of lin.
 * Every fp32 value is produced by the same operation sequence as the separate calls, so results are bit-identical.    */
#define DET_ACT_RMSNORM 1
#define DET_ACT_PLAIN 2
typedef struct {
    int kind;
    const float* a;
    const float* b;
    float eps;
    int8_t* xq;       /* optional outputs: all three or none */
    float* sx;
    uint16_t* mx;
    unsigned* amax;   /* DET_ACT_PLAIN only, may be NULL: the group maxima of a, see det_gemv_op.h_amax */
    /* Tensor parallel, may be NULL: a det_xchg handle.  The fp32 rows are then not read from memory: every rank's
     * local[M][slice] is exchanged as by det_xchg_all_gather (size * slice = K) and the gathered rows are the input.  With
     * kind DET_ACT_RMSNORM and acc_out != NULL, `a` is the residual stream: the normalized rows are a + gathered, and
     * acc_out (a buffer of its own, not `a`) receives those sums — det_xchg_add_rmsnorm_quant as the prologue of the GEMV
     * that consumes it.  Every rank must issue the same call; all rows go in one launch (M <= 8, M <= 2 with lin2).     */
    void* xchg;
    const float* local;
    int slice;
    float* acc_out;
} det_act_source;
typedef struct {
    const det_qlinear* lin;
    const det_qlinear* lin2;
    const det_act_source* src;
    const int8_t* xq;
    const float* sx;
    const uint16_t* mx;
    int M;
    float* y;                 /* outputs of lin, as det_gemm_ex: y / accumulate, or nparts / offs / dsts (host arrays) */
    int accumulate;
    int nparts;
    const int* offs;
    float* const* dsts;
    float* y2;                /* outputs of lin2 */
    int nparts2;
    const int* offs2;
    float* const* dsts2;
    float* h;
    /* With h, may be NULL: a buffer of 4 + 8 * M * (N/2)/128 words (16-byte aligned), zero before its first use.  The epilogue
     * folds max |h| of every 128-group into eight cells per group from word 4 on (fp32 bit patterns, integer atomic
     * maximum: order-free).  The det_gemv call that
     * quantizes h (src.kind = DET_ACT_PLAIN, src.a = h, src.amax = this buffer) reads them instead of scanning the rows,
     * which lifts the 8192-value limit of the prologue, and leaves the buffer zero again (word 0 counts its readers).
     * A buffer that was folded into must be consumed by exactly one such call (or cleared) before the next producer.  */
    unsigned* h_amax;
} det_gemv_op;
void det_gemv(const det_gemv_op* op, cudaStream_t st);

/* Seeded synthetic weights generated in device memory (the benchmarks' stand-in for a converted checkpoint; the host
 * twin is det_b200/csrc/host/synth.cpp and follows crates/det/src/quantize.rs:33-85).  det_synth_linear writes rows
 * [src_row0, src_row0 + n) of tensor `tid` of model `seed` into rows [row0, row0 + n) of a reference-layout linear
 * (wq, c, m as in det_qlinear); `scratch` needs n * (K/128) doubles.  det_synth_bf16 writes `count` bf16 elements.    */
void det_synth_linear(unsigned long long seed, unsigned long long tid, long long src_row0, int n, int K, int bits,
                      int row0, uint8_t* wq, float* c, uint16_t* m, double* scratch, cudaStream_t st);
/* Tensor-parallel helper: tmp[P][M][slice] (what an all-gather of per-rank [M][slice] blocks yields) -> full[M][P*slice]. */
void det_unshard(const float* tmp, float* full, int P, int M, int slice, cudaStream_t st);
void det_synth_bf16(unsigned long long seed, unsigned long long tid, long long count, uint16_t* out, cudaStream_t st);

/* Prefill attention on the tensor cores (batches of 16 tokens and more, head_dim 256, host-known position; the
 * reference's counterpart is the mma.sync path of kernels/cuda/attn.cu:405-852).  It stages the byte slices of the
 * probabilities and a transposed copy of V in a workspace the library allocates when it comes up (256 MB; the environment
 * variable DET_B200_ATTN_WS_MB changes the size, 0 = none).  det_attn_set_workspace replaces it with caller memory
 * (1024-byte aligned; NULL = none).  A call needs 512 * n_kv * Kpad bytes for V plus 512 * n_kv * Kpad bytes per tile of
 * 128 query rows (Kpad = keys rounded up to 128) and runs as many tiles per round as fit; without room for one tile the
 * call runs on the CUDA-core kernels.  Outputs are bit-identical either way.  det_debug_set_attn_tc: on = 0 switches the
 * tensor path off, min_m > 0 moves the batch threshold (measurement switch).                                          */
void det_attn_set_workspace(void* p, size_t bytes);
void det_debug_set_attn_tc(int on, int min_m);

/* Conversion and calibration on the device (the reference does both on the host: crates/det/src/convert.rs:346-369,
 * crates/det/src/quantize.rs:33-100, crates/det/src/calibrate.rs:21-36; crates/det/src/model.rs:389-413 for the table).
 * det_quantize_rows: `n` rows of K floats of a device tensor of ggml type 0 (F32), 1 (F16) or 30 (BF16) become det file
 * rows ([codes][c fp32][m u16 x K/128], crates/det/src/spec/tensor.rs:43-55) at rows_out; output row r reads source row
 * row_perm[r] (NULL: r) and its element k reads column col_perm[k] (NULL: k); `scratch` needs n * (K/128) doubles.  The
 * rows equal the host quantizer's byte for byte.
 * det_absmax_heads: slots[h] = max(slots[h], max |v[row][h][0..hd)|) over the t rows (slots start at zero; NaN skipped).
 * det_embed_table: det_embed for a table of ggml type 0, 1 or 30.                                                      */
void det_quantize_rows(const void* src, int ggml_type, const int* row_perm, const int* col_perm, int n, int K, int bits,
                       uint8_t* rows_out, double* scratch, cudaStream_t st);
void det_absmax_heads(const float* v, int t, int heads, int hd, float* slots, cudaStream_t st);
void det_embed_table(const void* table, int ggml_type, const int* ids, int M, int H, float* x, cudaStream_t st);

/* Decode-step graph (the reference lists "CUDA graphs for decode" as future work, README.md:115; its C side only has the
 * graph-capturable det_attention_dev).  det_graph_begin starts capturing everything issued on the library queue;
 * det_graph_end returns an executable graph (NULL on failure); det_graph_launch replays it on the queue.  Ops captured
 * this way must read their position from device memory (det_attention_dev) and their token from device memory
 * (det_embed with a device id).  Scratch buffers must have reached their final size before the capture starts.      */
void det_graph_begin(void);
void* det_graph_end(void);
void det_graph_launch(void* graph);
void det_graph_free(void* graph);
/* Token feedback of a replayed decode step: log[*pos - log_base] = *pick (when log != NULL and in range), then *pos += 1.
 * All pointers are device pointers.                                                                                  */
void det_token_feedback(const int* pick, int* pos, int* log, int log_base, int log_cap, cudaStream_t st);

/* Batched serving decode (no reference counterpart: its Model holds one sequence).  M sequences advance one token each;
 * row t of the activations belongs to the sequence whose cache / state is rows[t] — a DEVICE array of M structs — and,
 * for attention, whose position is pos[t] (device array; max_pos is a host bound on them; the caller guarantees
 * pos[t] < rows[t].capacity, which lives in device memory and is not checked here).  Row t equals
 * det_attention(M = 1, pos0 = pos[t]) / det_gdn(M = 1) on that sequence.  Scratch as for the single-sequence calls.  */
void det_attention_rows(const det_attn_layer* L, const det_kv_cache* rows, const int* pos, int max_pos, const float* qg,
                        const float* k, const float* v, const float* rope_cos, const float* rope_sin, int rot, float eps,
                        int M, int n_h, int n_kv, int hd, float* o, void* scratch, cudaStream_t st);
void det_gdn_rows(const det_gdn_layer* L, const det_gdn_state* rows, const float* qkv, const float* z, const float* a,
                  const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
                  cudaStream_t st);

/* Tensor-parallel exchange over NVLink peer memory (no reference counterpart: the reference is single-device).  Every
 * rank creates a staging area of the same size, publishes its CUDA IPC handle (64 bytes) and opens the others'.
 * det_xchg_all_gather sends local[M][slice] to every rank as self-validating 16-byte packets (plain peer stores) and
 * fills full[M][size*slice] — ordinary local memory, column block r = rank r's slice — as the packets of all ranks
 * arrive (bounded polling; a timeout sets the error word read by det_last_error).  One launch per rank, no host
 * involvement, capturable into the decode graph.  Every rank must issue the same sequence of exchanges, and the ranks
 * must pass a host barrier after det_xchg_open and before their first exchange: a receiver only waits for the wait limit
 * (about two seconds; det_debug_set_wait_limit), so a peer that is still loading its module or capturing its graph would
 * make the first exchange time out — the error word is then set, later reads return zeros at once, and det_clear_error
 * is the only way back.
 * `bytes` of staging take exchanges of up to det_xchg_capacity() gathered values (bytes / 16).                       */
void* det_xchg_create(size_t bytes, int rank, int size);
void det_xchg_ipc_handle(void* h, uint8_t out[64]);
void det_xchg_open(void* h, const uint8_t* handles /* size x 64 bytes */);
void det_xchg_open_loopback(void* h);   /* timing aid: all rank slots map to this rank's staging (values meaningless) */
size_t det_xchg_capacity(void* h);
void det_xchg_all_gather(void* h, const float* local, float* full, int M, int slice, cudaStream_t st);
void det_xchg_destroy(void* h);
/* The exchange fused with the row operation that consumes the gathered rows, n = size * slice.  All CTAs of such a launch
 * wait for packets of the other ranks, so they have to be resident together: det_xchg_fusable(M, n) says whether M rows of
 * n values qualify (single-token decode always does; a serving step of 32 rows does for rows up to 8192 values):
 *   det_xchg_add_rmsnorm_quant   gather local[M][slice]; x[M][n] += gathered; det_rmsnorm_quant(x, w) -> xq, sx, mx
 *   det_xchg_quant               gather local (or silu(local) * local_b when local_b != NULL); det_quant -> xq, sx, mx
 * Results equal det_xchg_all_gather followed by det_add / det_rmsnorm_quant / det_silu_mul_quant / det_quant.       */
int det_xchg_fusable(int M, int n);
void det_xchg_add_rmsnorm_quant(void* h, const float* local, int slice, float* x, const float* w, float eps, int M,
                                int8_t* xq, float* sx, uint16_t* mx, cudaStream_t st);
void det_xchg_quant(void* h, const float* local, const float* local_b, int slice, int M, int8_t* xq, float* sx,
                    uint16_t* mx, cudaStream_t st);

/* No counterpart in the reference.  det_sample_topkp for callers that may not allocate device memory (hosts that fix
 * their memory budget at start-up, plug-ins that are only handed pointers): the weight scratch is a fixed 4 MiB array
 * inside the library, so there is no scratch argument and no allocation of any kind inside the call.  Limit: M * V <=
 * 524288 whenever top-k or top-p is active; a request without an active filter needs no scratch and is taken at any size.
 * Returns 0 when the work was queued, 1 when the request was refused (too large, V <= 0, det_init never called) or the
 * launch was rejected; a refusal prints its reason and launches nothing; the call never aborts.  The first call on a
 * device resolves the array's address (and makes the driver load the module holding it): make it at start-up, outside
 * stream capture.  Calls share the array, so calls that overlap on the GPU race.                                       */
int det_sample_topkp_static(const float* logits, int M, int V, float inv_temp, int top_k, float top_p,
                            const unsigned long long* z, int* out, cudaStream_t st);

/* Measurement switch: programmatic dependent launch between the library's kernels on (default, non-zero) or off.
 * Results are identical either way; only the overlap of one kernel's prologue with its predecessor's tail changes.  */
void det_debug_set_pdl(int on);
/* Measurement switch for the row kernels: calls with at least min_rows rows (default 128; 0 = never) use one CTA per row
 * instead of a cluster per row.  Same results.                                                                       */
void det_debug_set_rows(int min_rows);
/* Measurement switch: pins the tensor-core GEMM's tile, 1 / 2 / 3 = 32 / 64 / 128 tokens per CTA; 0 = chosen by shape
 * (default).  Adding 0x100 / 0x200 switches the split of K over several CTAs for linears with few row tiles on / off.
 * Results do not depend on any of it.                                                                                 */
void det_debug_set_tc_variant(int v);
/* Measurement switch of the decode GEMV: bits 4..8 = worker warps per CTA (0 = all sixteen); bits 9.. = shared-memory
 * slots per worker warp (0 = as many as fit, at most 5).  Results do not depend on it.                                */
void det_debug_set_gemv(int flags);
/* Tensor-pipe ceiling: tcgen05.mma kind::i8 (128 x 256 x 32) issued back to back from resident shared-memory tiles on
 * every SM, no loads and no epilogue; returns the measured int8 rate in TOPS.                                         */
double det_debug_umma_peak(int iters);
/* Transport ceiling of a weight stream: `reps` launches that each read `bytes` of device memory with nothing to compute
 * (launch r reads piece r % regions of a buffer of regions * bytes; launches chained by programmatic dependent launch);
 * returns GB/s (events on the library queue).  mode 0 = plain 16-byte loads, grid-stride; mode 1 = the decode GEMV's transport (one
 * CTA per SM, `warps` warps with `slots` shared-memory slots each, records of rec_bytes by cp.async.bulk, nch consecutive
 * records per quad, quads dealt round-robin over CTAs and warps); mode 2 = the same ring over one contiguous span per
 * CTA.  regions * bytes well above the L2 size measures HBM.                                                                */
double det_debug_stream_peak(const void* p, size_t bytes, int regions, int mode, int rec_bytes, int warps, int slots,
                             int nch, int reps);

/* Last error recorded by a bounded device-side wait (0 = none, 1 = a wait ran out, 2 = a size check failed on the
 * device).  Waits for pending work.  While the word is set, exchange waits return at once (with zeros) instead of
 * polling, so a caller that has dealt with the error clears it with det_clear_error before it carries on.  Ranks of a
 * tensor-parallel group must pass a host barrier before their first exchange (a start-up skew longer than the wait limit
 * would otherwise expire the first wait).                                                                            */
int det_last_error(void);
void det_clear_error(void);
/* Limit of every bounded device-side wait (mbarrier waits of the GEMM kernels, packet polls of the exchange, the counter
 * of the fused decode attention) in SM clock cycles; <= 0 restores the default of 4e9 (about two seconds).  With
 * det_debug_xchg_drop — loopback exchange handles only: column block `rank` is no longer sent, rank < 0 undoes it — a
 * test can make a wait run out without faulting or hanging anything.                                                  */
void det_debug_set_wait_limit(long long cycles);
void det_debug_xchg_drop(void* h, int rank);

#ifdef __cplusplus
}
#endif
#endif /* DET_B200_H */
