// Internal launcher interface between the C ABI (api.cu), the Llama2 host plumbing (engine.cu)
// and the kernel files. Every launcher only enqueues on `st` and returns a tl_status.
#pragma once

#include "common.cuh"

namespace tlb {

// ---- runtime.cu: lookup tables computed on the host with the reference's own formulas ---------
struct Tables {
    const __half* exp_tab;         // [65536] half(exp((double)float(h)))        softmax.cpp:22
    const __half* silu_float_tab;  // [65536] SiLU through float                 CPU.cpp:220-222
    const __half* silu_half_tab;   // [65536] SiLU fp16 route as shipped         CPU.cpp:216-219
};
const Tables& tables();
// int32 in device memory, 0 unless a kernel gave up on a bounded wait (then a tl_status code)
int* device_status_word();
// turn a host copy of the status word (fetched at a sync point) into a return code; clears the word
int consume_device_status(int value);
// cos/sin tables [rows, head_dim/2] for positions [0, rows); grows on demand by allocating a larger
// generation. Pointers handed out earlier stay valid for the life of the process.
int rope_table(int head_dim, int min_rows, const __half** cos_t, const __half** sin_t);

// ---- ops_refmode.cu: reference-order kernels (bit-identical to the reference CPU backend) ----
// C_b(m,n) = sum_k A_b(m,k) * B_b(n,k), k ascending, fp32 accumulate, one rounding; arbitrary
// element strides (a_m,a_k / b_n,b_k / c_m; C is contiguous along n) and batch strides.
struct SeqMatmul {
    const __half* A; const __half* B; __half* C;
    int batch, M, N, K;
    long long a_m, a_k, b_n, b_k, c_m, sA, sB, sC;
};
int launch_matmul_seq(const SeqMatmul& p, cudaStream_t st);
int launch_rmsnorm_seq(__half* out, const __half* in, const __half* w, float eps, int hidden,
                       int tokens, cudaStream_t st);
int launch_softmax_seq(__half* out, const __half* in, size_t rows, size_t cols, cudaStream_t st);
// scores (H,T,S): e = e / half(sqrt(head_dim)); if T > 1: e += (s > pos + t ? -inf : 0)
int launch_scale_mask(__half* scores, int H, int T, int S, int pos, int head_dim, cudaStream_t st);

// ---- elementwise / gather / argmax (same in both numerics) ------------------------------------
int launch_rope(const __half* in, __half* out, int start_pos, int rows_bt, int T, int n_heads,
                int head_dim, const __half* cos_t, const __half* sin_t, cudaStream_t st);
int launch_silu(__half* out, const __half* in, size_t n, int via_float, cudaStream_t st);
int launch_binary(__half* out, const __half* a, const __half* b, size_t n, int op, cudaStream_t st);
int launch_div_scalar(__half* out, const __half* a, __half scalar, size_t n, cudaStream_t st);
int launch_argmax(int* out_idx, const __half* in, size_t rows, size_t cols, cudaStream_t st);
int launch_embedding(__half* out, const __half* table, const int* tokens, int n_tokens, int dim,
                     int vocab, cudaStream_t st);
// rows of `dim` halfs: dst[(dst_row0 + r) * dst_pitch ...] = src[r * dim ...]
// out[i] = a[i] + half(sum32[i]) in fp16 (a K-split matmul's reduced sum, then the residual add)
int launch_residual_add_f32(__half* out, const __half* a, const float* sum32, size_t n, cudaStream_t st);
int launch_copy_rows(__half* dst, const __half* src, int rows, int dim, long long dst_pitch,
                     cudaStream_t st);

// ---- device_ops.cu: the rest of the Device<half> surface ------------------------------------------
int launch_contiguous(__half* result, const __half* data, const int* shape, const int* stride, int ndim, size_t offset,
                      size_t n, cudaStream_t st);
int launch_set_item(__half* data, const __half* src, const int* shape, const int* stride, int ndim, size_t offset,
                    size_t n, cudaStream_t st);
int launch_set_item_scalar(__half* data, __half value, const int* shape, const int* stride, int ndim, size_t offset,
                           size_t n, cudaStream_t st);
int launch_unary(__half* out, const __half* in, size_t n, int op, cudaStream_t st);
int launch_binary_op(__half* out, const __half* a, const __half* b, size_t n, int op, cudaStream_t st);
int launch_binary_scalar(__half* out, const __half* a, __half s, size_t n, int op, cudaStream_t st);
int launch_reduce(__half* out, const __half* in, size_t reduce_size, size_t n, int op, int numerics, cudaStream_t st);
int launch_argreduce(int* out_idx, const __half* in, size_t reduce_size, size_t n, int want_min, cudaStream_t st);
int launch_cast(void* out, const void* in, size_t n, int kind, cudaStream_t st);

// ---- gemv.cu: the decode path (M = 1..8), fast numerics ---------------------------------------
// y[m, n] = sum_k x[m, k] W[n, k]; requires K % 8 == 0 and 16-byte aligned rows.
bool gemv_supported(const void* x, const void* W, size_t M, size_t N, size_t K, size_t ldw);
// weights_constant: no kernel in flight on `st` writes W, so its stream may start before the previous
// kernel of the stream has finished (nn::Linear's parameter; a generic matmul operand may not promise that)
int launch_gemv(const __half* x, const __half* W, __half* y, int M, int N, int K, long long ldw,
                long long ldx, long long ldy, cudaStream_t st, bool weights_constant = false);
// 2 <= M <= 8 on the weight-streaming ring (the activation rows are the columns of the MMA's B operand)
bool gemv_ring_rows_supported(const void* x, const void* W, size_t M, size_t N, size_t K, size_t ldw, size_t ldx);

enum GemvEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_QKV_ROPE = 2, EPI_SWIGLU = 3, EPI_STORE_F32 = 4,
                    EPI_PUSH_F32 = 5, EPI_PUSH_F16 = 6 };

// Tensor-parallel exchange fused into the GEMV kernels (no collective library call in between).
// Producer side (a K-split matmul: wo, w2; or the vocabulary-split classifier): the epilogue
// stores its results straight into slot [my_rank] of a receive buffer in EVERY rank's memory
// (plain peer stores over NVLink). Every 8-byte word carries 4 bytes of payload (one fp32
// partial sum, or two fp16 logits) and the 4-byte epoch of this step and phase, written by one
// 8- or 16-byte store, so a word is valid exactly when its epoch matches: no flags, no fences,
// no counters, and the latency of an exchange is one store's flight over NVLink.
// Consumer side (the prologue of the next GEMV): read the `world` slots, retry (bounded) any
// word whose epoch is not this step's yet, sum in rank order in fp32, round once to fp16 and add
// the residual in fp16, i.e. the arithmetic of the single-GPU path up to fp32 summation order.
// Data is pushed into the consumer's own memory; nothing is ever loaded from a peer.
// Slots are reused every step without a second handshake: a rank can only reach the next writer
// of a slot after consuming data its peers produce after their reads of that slot.
constexpr int TL_MAX_TP = 8;
// Polls a consumer spends on words that have not arrived before it gives up (each poll is a round of
// L2 reads, 0.5-1 us): about two seconds, long enough for a rank that was held up on the host by an
// allocation or a graph instantiation, short enough that a lost rank surfaces as TL_ERR_TIMEOUT.
constexpr unsigned int TL_EXCHANGE_TRIES = 1u << 21;
struct PeerExchange {
    int world, rank;
    int n;                                       // payload elements per rank slot (fp32 sums or fp16 logits)
    const unsigned long long* local_slots;       // consumer view: [world][words per slot]
    unsigned long long* local_pub;               // consumer side: [n / 2] (two halfs, epoch) words, the reduced vector published once per GPU
    unsigned long long* peer_slot[TL_MAX_TP];    // producer view: slot [my rank] in rank d's memory
    const unsigned int* step_ptr;                // local: decode step counter (same value on every rank)
    int phases_per_step, phase_id;               // epoch = *step_ptr * phases_per_step + phase_id + 1
    // consumer extras
    const __half* residual; __half* sum_out;     // x = residual + sum; CTA 0 also writes it to sum_out
    // 1: every CTA sums the ranks' slots itself (world x n words of L2 reads per CTA, no publish / gather hop);
    // 0: CTA c sums slice c and publishes it, every CTA gathers the published vector (one more on-chip hop, n / 2 words per CTA)
    int direct;
};
struct FusedGemv {
    // input vector (M = 1) and optional RMSNorm prologue
    const __half* x;            // [K]
    const __half* norm_w;       // [K] or nullptr: no norm
    float eps;
    // up to three weight matrices [N_each, K] sharing x (wq|wk|wv, w1|w3, or a single one)
    const __half* W[3];
    int n_mats, N_each, K;
    int epilogue;
    // EPI_STORE / EPI_RESIDUAL: y[n] (+ residual[n])
    __half* y; const __half* residual;
    float* y32;                 // EPI_STORE_F32: unrounded fp32 sums (partial sums of a K-split matmul)
    // EPI_QKV_ROPE: q -> y, k -> k_out, v -> v_out (rows of the caches at the current position)
    __half* k_out; __half* v_out; const __half* cos_row; const __half* sin_row; int head_dim;
    // position-dependent pointers when replayed from a CUDA graph: if pos_ptr != nullptr the
    // kernel adds (*pos_ptr) * kv_pitch to k_out / v_out and (*pos_ptr) * head_dim/2 to cos/sin
    const int* pos_ptr; long long kv_pitch;
    bool pdl;                   // launch with programmatic stream serialization
    bool weights_may_change;    // the previous kernel of the stream may have written W: stream it after the wait
    const PeerExchange* xin;    // prologue: x = residual + sum over ranks of a pushed partial vector
    unsigned long long* prof;   // optional device buffer for three %globaltimer stamps of CTA 0 (start, vector staged, done)
    unsigned int xin_tries;     // 0: the default bound on the polls of that wait (TL_EXCHANGE_TRIES)
    const PeerExchange* xout;   // EPI_PUSH_F32 / EPI_PUSH_F16: where the results go on every rank
};
int launch_fused_gemv(const FusedGemv& p, cudaStream_t st);
// two phases in one launch: a K-split matmul that pushes its partial sums, then the matmul that consumes the exchanged sum
int launch_fused_gemv_pair(const FusedGemv& a, const FusedGemv& b, cudaStream_t st);

// ---- attn.cu: attention, fast numerics -----------------------------------------------------------
struct DecodeAttn {
    const __half* q;        // [H, hd]
    const __half* k_cache;  // [S_max, H, hd]
    const __half* v_cache;
    __half* out;            // [H, hd]
    float* scratch;         // [H, splits, hd + 2] fp32 partials
    unsigned int* counters; // [H] zero before the first launch; the kernel re-zeroes them
    int H, head_dim, seq_len /* positions 0..seq_len-1 are attended */, splits;
    const int* pos_ptr;     // if set: seq_len = *pos_ptr + 1
    long long kv_pitch;     // elements between consecutive positions (H*hd of this rank)
    bool pdl;
};
int launch_decode_attn(const DecodeAttn& p, cudaStream_t st);
// the same with the splits of a head merged over distributed shared memory (cluster of <= 8 CTAs);
// scratch and counters are not used
int launch_decode_attn_cluster(const DecodeAttn& p, cudaStream_t st);
// causal softmax over materialised scores (H,T,S) with scale, fp32 internals, in place
int launch_softmax_causal_fast(__half* scores, int H, int T, int S, int pos, float scale,
                               cudaStream_t st);
int launch_rmsnorm_fast(__half* out, const __half* in, const __half* w, float eps, int hidden,
                        int tokens, cudaStream_t st);
int launch_softmax_fast(__half* out, const __half* in, size_t rows, size_t cols, cudaStream_t st);
// out[i] = silu(gate[i]) * up[i] (fp32 internals); residual add
int launch_swiglu_fast(__half* out, const __half* gate, const __half* up, size_t n, cudaStream_t st);
// vt[h, d, s] = v[s, h, d] for s in [0,S)
int launch_transpose_v(__half* vt, const __half* v, int S, int H, int hd, long long v_pitch,
                       long long vt_pitch_s, cudaStream_t st);

// ---- attn_sm100.cu: prefill attention on tcgen05 / TMEM / TMA (head_dim 128) ----------------------
bool flash_prefill_supported(const void* q, const void* k, const void* v, const void* out, int T, int S, int pos0,
                             int heads, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo);
int launch_flash_prefill(const __half* q, const __half* k, const __half* v, __half* out, int T, int S, int pos0,
                         int heads, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                         cudaStream_t st);
bool tensor_map_encode_available();

// ---- hgemm_sm100.cu: prefill HGEMM on tcgen05 / TMEM / TMA -----------------------------------------
bool hgemm_supported(const void* A, const void* B, const void* C, size_t M, size_t N, size_t K,
                     size_t lda, size_t ldb, size_t ldc);
// true when the cluster split-K HGEMM has a plan for this shape (few tiles, long K): callers prefer it to the
// skinny kernel for 9..128 rows
bool hgemm_splitk_preferred(int M, int N, int K);
// weights_constant: B is never written by another kernel of the stream (a model weight), so a kernel may
// request its first tiles before the programmatic-dependency wait
int launch_hgemm(const __half* A, const __half* B, __half* C, int batch, int M, int N, int K,
                 long long lda, long long ldb, long long ldc, long long sA, long long sB,
                 long long sC, cudaStream_t st, bool weights_constant = false);

// K-split matmul of the tensor-parallel prefill: C[M, N] is this rank's partial result, stored locally; the rank
// that owns rows [o * rows_per_owner, (o + 1) * rows_per_owner) is told when it may fetch them: after a 128-row x
// tile-width piece is stored, flags[owner][(m0 % rows_per_owner) / 128 * 64 + column tile] = epoch (a 4-byte peer
// store). *col_tiles returns how many column tiles (flags per row block) the chosen kernel produces.
struct HgemmPush {
    int world, rows_per_owner;
    unsigned int epoch;
    unsigned int* flags[TL_MAX_TP];    // this rank's flag block in rank d's memory
};
int launch_hgemm_push(const __half* A, const __half* B, __half* C, int M, int N, int K, long long lda, long long ldb,
                      const HgemmPush& push, int* col_tiles, cudaStream_t st);
// The owner's side: rows [0, rows) of this rank's slice = residual + sum over source ranks (rank order, fp32) of
// their partial rows, fetched from the sources' memory (plain peer loads, a warp reads 512 contiguous bytes) once
// every (row block, column tile) flag of every source reads `epoch`; the new residual rows are written locally,
// their RMSNorm (times norm_w) is stored into row (row0 + r) of xn_dst[d] on every rank d; when the last row of
// the slice is done (counted in *rows_done, left at 0) owner_done[d][rank] = epoch on every rank d. Bounded waits
// (TL_ERR_TIMEOUT in the status word).
struct TpReduceNorm {
    int world, rank, rows, row0, dim, col_tiles;
    unsigned int epoch;
    const __half* partial[TL_MAX_TP];  // rank s's partial result [T][dim] (peer pointer; s = this rank: local)
    const unsigned int* arrive_flags;  // [world][row blocks][64], local
    int flags_slot_stride;             // words between two sources' flag blocks
    const __half* residual;            // local rows [row0, row0 + rows) x dim
    __half* residual_out;
    const __half* norm_w; float eps;
    __half* xn_dst[TL_MAX_TP];
    unsigned int* owner_done[TL_MAX_TP];   // [world] flag words in rank d's memory
    unsigned int* rows_done;               // local counter, 0 between exchanges
};
int launch_tp_reduce_norm(const TpReduceNorm& p, cudaStream_t st);
// wait (bounded) until row flags [0, rows) read `epoch`: every owner's normalised rows have arrived here
int launch_tp_wait_owners(const unsigned int* flags, int owners, unsigned int epoch, cudaStream_t st);

// ---- skinny_sm100.cu: 2 <= M <= 128, weights streamed once (swap-AB tcgen05, stream-K split) --------
bool skinny_supported(const void* A, const void* W, size_t M, size_t N, size_t K, size_t lda, size_t ldw);
struct SkinnyPlan { int nb, tiles, nkb, per, grid, cluster_splits; };
SkinnyPlan skinny_plan(int M, int N, int K, int sms);
int launch_skinny(const __half* A, const __half* W, __half* C, int M, int N, int K, long long lda, long long ldw,
                  long long ldc, cudaStream_t st, bool weights_constant = false);

// which tile the plain HGEMM would use on `sms` SMs: kind 0 = single-CTA tile of width *bn, 1 = CTA-pair 256x256
void hgemm_plan(int M, int N, int K, int batch, int sms, int* kind, int* bn, int* sk_per);

// fused epilogues of the prefill HGEMM (N % 32 == 0, 16-byte aligned rows)
bool hgemm_fused_supported(const void* A, const void* B, const void* C, size_t M, size_t N, size_t K, size_t lda,
                           size_t ldb, size_t ldc);
int launch_hgemm_residual(const __half* A, const __half* B, const __half* R, __half* C, int M, int N, int K,
                          long long lda, long long ldb, long long ldr, long long ldc, cudaStream_t st,
                          bool weights_constant = false);
int launch_hgemm_swiglu(const __half* A, const __half* W1, const __half* W3, __half* C, int M, int N, int K,
                        long long lda, long long ldb, long long ldc, cudaStream_t st);
int launch_hgemm_qkv_rope(const __half* A, const __half* Wq, const __half* Wk, const __half* Wv, __half* q_out,
                          __half* k_rows, __half* v_rows, int M, int n_each, int K, long long lda, long long ldb,
                          long long ldq, long long ld_kv, const __half* cos_rows, const __half* sin_rows,
                          int head_dim, cudaStream_t st);

}  // namespace tlb
