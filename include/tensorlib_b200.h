/*
 * tensorlib_b200 — C ABI of the B200 (sm_100a) matmul backend for tensorLib's
 * Tensor::matmul -> Llama2 forward path.
 *
 * Conventions
 *   - fp16 values are IEEE binary16 bit patterns (tl_half). Unless a parameter is named
 *     *_host, every pointer is a DEVICE pointer on the device chosen by tl_init().
 *   - Every function returns a tl_status (0 = TL_OK); nothing prints or exits. The message of
 *     the last failure on the calling thread is returned by tl_last_error().
 *   - Functions taking a tl_stream only enqueue work on that cudaStream_t (NULL = the legacy
 *     default stream, which is what the reference uses everywhere) and return without
 *     synchronising, unless stated.
 *   - There is no CPU fallback: without a usable sm_100 device tl_init() fails and every
 *     compute entry point returns TL_ERR_NOT_INITIALIZED.
 *   - `numerics` selects the summation order, never the storage type (always fp16 in, fp32
 *     accumulate, fp16 out):
 *       TL_NUMERICS_REFERENCE_ORDER  the rounding points and the sequential accumulation order
 *                                    of the reference's CPU backend; results are bit-identical
 *                                    to it. Slow (dependent chains), meant for parity runs.
 *       TL_NUMERICS_FAST             parallel fp32 reductions / tensor cores.
 *
 * Each declaration cites the reference interface it replaces (paths inside DavidZyy/tensorLib).
 */
#ifndef TENSORLIB_B200_H
#define TENSORLIB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TL_API __attribute__((visibility("default")))
#else
#define TL_API
#endif

typedef uint16_t tl_half;
typedef void* tl_stream; /* cudaStream_t */

typedef enum tl_status {
    TL_OK = 0,
    TL_ERR_INVALID_ARGUMENT = 1, /* the reference throws std::invalid_argument here */
    TL_ERR_NOT_INITIALIZED = 2,
    TL_ERR_CUDA = 3,             /* the reference prints and exit(1)s here (CUDA.cuh:131-151) */
    TL_ERR_UNSUPPORTED = 4,
    TL_ERR_OUT_OF_MEMORY = 5,
    TL_ERR_TIMEOUT = 6,          /* a bounded device-side wait gave up */
    TL_ERR_COMM = 7,
    TL_ERR_IO = 8
} tl_status;

enum { TL_NUMERICS_REFERENCE_ORDER = 0, TL_NUMERICS_FAST = 1 };

/* ---- library ---------------------------------------------------------------------------- */
TL_API const char* tl_strerror(int status);
TL_API const char* tl_last_error(void);
TL_API int tl_version(void);
/* Select `device`, verify it is sm_100, make it current for the calling thread. */
TL_API int tl_init(int device);
TL_API int tl_device_count(int* count);
/* Synchronise the device and fetch (then clear) the device status word: 0, or TL_ERR_TIMEOUT if a
 * kernel gave up on one of its bounded waits (mbarrier polls). The reference has no counterpart:
 * its kernels never wait on anything. */
TL_API int tl_device_status(int* status);

/* Host-only introspection of the lookup tables the kernels use for exp / SiLU / RoPE. They are
 * evaluated on the host with the formulas of the reference's CPU backend (cpu/softmax.cpp:22,
 * CPU.cpp:216-222, CPU.cpp:444-447); each *_tab has 65536 entries indexed by the fp16 bit
 * pattern; the rope tables are [rows, head_dim/2]. No device needed. */
TL_API int tl_host_lookup_tables(tl_half* exp_tab, tl_half* silu_float_tab, tl_half* silu_half_tab);
TL_API int tl_host_rope_table(int head_dim, int rows, tl_half* cos_out, tl_half* sin_out);

/* ---- device memory: what CUDA<dtype>'s ctor/dtor and getData/setData do
 *      (tensorLib/src/device/cuda/CUDA.cu:17-32, :72-81) -------------------------------------- */
TL_API int tl_malloc(void** dptr, size_t bytes);
TL_API int tl_free(void* dptr);
TL_API int tl_memcpy_h2d(void* dst, const void* src_host, size_t bytes, tl_stream stream);
TL_API int tl_memcpy_d2h(void* dst_host, const void* src, size_t bytes, tl_stream stream);
TL_API int tl_memcpy_d2d(void* dst, const void* src, size_t bytes, tl_stream stream);
TL_API int tl_memset(void* dst, int value, size_t bytes, tl_stream stream);
TL_API int tl_stream_synchronize(tl_stream stream);
TL_API int tl_malloc_host(void** hptr, size_t bytes); /* pinned */
TL_API int tl_free_host(void* hptr);

/* ---- matmul: the drop-in boundary --------------------------------------------------------- */
/* Device<half>::matmul2d (tensorLib/include/device/Device.hpp:22; CUDA implementation
 * tensorLib/src/device/cuda/gemm.cu:153-172): C[M,N] = A[M,K] * B[N,K]^T, all row-major
 * contiguous. Dispatches on M in fast numerics: M = 1..8 the streaming GEMV ring (up to eight
 * activation rows ride the eight columns of the MMA's B operand, so they cost the weight traffic
 * of one; needs N even and K % 16 == 0), 9..128 (and other 2..8 shapes) the skinny tensor-core
 * kernel (weights streamed once), larger M the tcgen05 HGEMM (single-CTA or CTA-pair tiles);
 * operands that are not 16-byte aligned or K % 8 != 0 take the any-shape kernel.
 * All kernels are launched with programmatic stream serialization and wait on the device for the
 * previous kernel of `stream` before touching A, B or C, so back-to-back calls overlap their
 * set-up, never their data. The first skinny call on a given stream allocates a 34 MB workspace
 * for that stream (kept until exit): make it before starting a stream capture. */
TL_API int tl_matmul2d_f16(const tl_half* A, const tl_half* B, tl_half* C, size_t M, size_t N, size_t K,
                    int numerics, tl_stream stream);
/* nn::Linear<half>::forward (tensorLib/src/nn/linear.cpp:43-49; weight [out, in] as linear.cpp:10-14
 * stores it): y[T, out] = x[T, in] * W[out, in]^T in fast numerics. Same kernels as tl_matmul2d_f16
 * with one more promise from the caller: W is a parameter, i.e. no kernel in flight on `stream`
 * writes it. For T <= 8 the weight stream then starts before the previous kernel of the stream has
 * finished (only x and y are ordered behind it), which takes the ring's fill latency off a chain of
 * Linear layers. */
TL_API int tl_linear_f16(const tl_half* x, const tl_half* W, tl_half* y, size_t T, size_t in_features,
                         size_t out_features, tl_stream stream);
/* The per-batch loop of ops::matmul::call2 (tensorLib/src/ops/matmul.cpp:297-321) as one call:
 * for b in [0,batch): C_b[M,N] = A_b[M,K] * B_b[N,K]^T with row pitches lda/ldb/ldc and batch
 * strides (all in elements; a batch stride of 0 broadcasts, as call2's stride-0 views do). */
TL_API int tl_matmul_batched_f16(const tl_half* A, const tl_half* B, tl_half* C, size_t batch, size_t M,
                          size_t N, size_t K, size_t lda, size_t ldb, size_t ldc, size_t strideA,
                          size_t strideB, size_t strideC, int numerics, tl_stream stream);
/* Device<half>::matmul, the strided batched form (tensorLib/include/device/Device.hpp:13-20; CUDA
 * form tensorLib/src/device/cuda/gemm.cu:28-85, CPU form CPU.cpp:18-68): result is contiguous with
 * shape result_shape[ndim] = (batch dims..., M, N); element (b..., m, k) of lhs sits at
 * lhs[lhs_offset + sum_i b_i*lhs_stride[i] + m*lhs_stride[ndim-2] + k*lhs_stride[ndim-1]], element
 * (b..., k, n) of rhs at rhs[rhs_offset + sum_i b_i*rhs_stride[i] + k*rhs_stride[ndim-2] +
 * n*rhs_stride[ndim-1]] (a stride of 0 broadcasts). This is the call the legacy op
 * ops::matmul::call makes (matmul.cpp:18-93). When the reduction dimension is contiguous in both
 * operands (what Linear and the attention matmuls produce) fast numerics runs the same kernels as
 * tl_matmul_batched_f16, one launch per innermost batch dimension; any other layout runs the
 * any-stride kernel, which also is the reference-order path (sequential fp32 sum over k, one rounding,
 * like the reference's CPU code; the reference's CUDA kernel accumulates in half). */
TL_API int tl_matmul_strided_f16(const tl_half* lhs, const tl_half* rhs, tl_half* result, const int* lhs_stride_host,
                                 const int* rhs_stride_host, size_t lhs_offset, size_t rhs_offset,
                                 const int* result_shape_host, int ndim, size_t result_elements, size_t K, int numerics,
                                 tl_stream stream);
/* Host-only introspection (no device needed): the kernel tl_matmul2d_f16 selects in fast numerics for
 * 16-byte aligned operands on a device with sm_count SMs, and how the work is cut: CTAs launched,
 * tile width along N (the padded batch for the skinny kernels), k-blocks of 64 per CTA (skinny
 * kernels) or per CTA pair (the pair kernel's stream-K mode; 0 = whole tiles), CTAs per cluster
 * (0 = no clusters). */
enum { TL_PLAN_REFERENCE_ORDER = 0, TL_PLAN_GEMV_RING = 1, TL_PLAN_GEMV_SMALL = 2, TL_PLAN_SKINNY_STREAMK = 3,
       TL_PLAN_SKINNY_CLUSTER = 4, TL_PLAN_HGEMM = 5, TL_PLAN_HGEMM_PAIR = 6 /* 256-row tiles per CTA pair */,
       TL_PLAN_HGEMM_PAIR512 = 7 /* 512-row tiles per CTA pair */,
       TL_PLAN_HGEMM_SPLITK = 8 /* one 128-row tile per cluster, K split over its CTAs (cluster = CTAs per tile) */ };
TL_API int tl_matmul_plan(size_t M, size_t N, size_t K, int sm_count, int* kernel, int* grid, int* tile_n,
                   int* k_blocks_per_cta, int* cluster);
/* Same contract as tl_matmul2d_f16 with HOST buffers: copies A and B in, C out, synchronises. */
TL_API int tl_matmul2d_f16_host(const tl_half* A_host, const tl_half* B_host, tl_half* C_host, size_t M,
                         size_t N, size_t K, int numerics);

/* ---- the operators next to a matmul in the Llama2 forward --------------------------------- */
/* CUDA<half>::rms_norm (tensorLib/include/device/cuda/CUDA.cuh:108, rms_norm.cu:181-184; CPU
 * semantics nn::RMSNorm::forward_plain, tensorLib/src/nn/rmsNorm.cpp:15-56). */
TL_API int tl_rms_norm_f16(tl_half* out, const tl_half* in, const tl_half* weight, float eps, int hidden,
                    int tokens, int numerics, tl_stream stream);
/* Device::apply_rotary_emb (Device.hpp:91-98, CPU.cpp:427-461): interleaved-pair rotation of a
 * contiguous (B,T,n_heads,head_dim) tensor; in == out allowed. cos/sin come from a table
 * computed on the host with the reference's float formula, so both numerics agree bit for bit.
 * When start_pos+T exceeds what earlier calls needed, a larger table is allocated and filled (a
 * blocking copy); tables handed out before, e.g. to a model, stay allocated and valid. */
TL_API int tl_apply_rotary_emb_f16(const tl_half* in, tl_half* out, int start_pos, int B, int T,
                            int n_heads, int head_dim, tl_stream stream);
/* Device::softmax over the last dimension (Device.hpp:77, cpu/softmax.cpp:10-31). */
TL_API int tl_softmax_f16(tl_half* out, const tl_half* in, size_t rows, size_t cols, int numerics,
                   tl_stream stream);
/* Device::silu (Device.hpp:57). via_float = 1: x*sigmoid(x) in fp32, one rounding (the
 * reference's CUDA kernel, CUDA.cu:334-342, and its CPU float route). via_float = 0: the CPU
 * fp16 route as shipped, including its 1/(1+exp(x)) sign defect (CPU.cpp:216-219). */
TL_API int tl_silu_f16(tl_half* out, const tl_half* in, size_t n, int via_float, tl_stream stream);
/* Device::add / mul / div-by-scalar (Device.hpp:62-70). */
TL_API int tl_add_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, tl_stream stream);
TL_API int tl_mul_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, tl_stream stream);
TL_API int tl_div_scalar_f16(tl_half* out, const tl_half* a, double scalar, size_t n, tl_stream stream);
/* Device::argmax over the last dimension (Device.hpp:75, CPU.cpp:358-372): the LOWEST index
 * wins ties. out_idx: int32[rows]. */
TL_API int tl_argmax_f16(int* out_idx, const tl_half* in, size_t rows, size_t cols, tl_stream stream);
/* nn::Embedding::forward (tensorLib/src/nn/embedding.cpp:48-81): out[t,:] = table[tokens[t],:],
 * token ids read from device memory. */
TL_API int tl_embedding_f16(tl_half* out, const tl_half* table, const int* tokens, int n_tokens, int dim,
                     int vocab, tl_stream stream);

/* ---- the rest of the Device<half> surface (tensorLib/include/device/Device.hpp:30-78) -----------
 * What an arbitrary Tensor<half> program needs from its device besides matmul. Arithmetic follows
 * the reference's CPU backend bit for bit (tensorLib/src/device/cpu/CPU.cpp:127-402) except where
 * noted; the kernels replace tensorLib/src/device/cuda/CUDA.cu:83-210, :440-464, binary.cuh:42-75
 * and reduce.cuh:18-39. All are stream-ordered and return without synchronising. */
/* Device::contiguous / setItemEwise / setItemScalar (Device.hpp:30-47): element i of the logical
 * row-major order of `shape` lives at data[offset + sum_d idx_d * stride[d]] (convertIdx,
 * CUDA.cuh:186-202). shape / stride: `ndim` <= 8 host ints (strides may be 0 for a broadcast view
 * being read); n = product of shape < 2^32.
 *   tl_contiguous_f16     result[i] = data[strided(i)]
 *   tl_set_item_f16       data[strided(i)] = src[i]
 *   tl_set_item_scalar_f16 data[strided(i)] = value */
TL_API int tl_contiguous_f16(tl_half* result, const tl_half* data, const int* shape_host, const int* stride_host,
                             int ndim, size_t offset, size_t n, tl_stream stream);
TL_API int tl_set_item_f16(tl_half* data, const tl_half* src, const int* shape_host, const int* stride_host, int ndim,
                           size_t offset, size_t n, tl_stream stream);
TL_API int tl_set_item_scalar_f16(tl_half* data, tl_half value, const int* shape_host, const int* stride_host, int ndim,
                                  size_t offset, size_t n, tl_stream stream);
/* Device::neg .. rsqrt (Device.hpp:49-58, CPU.cpp:169-276): out[i] = f(in[i]), evaluated as the
 * reference does (to float, libm function, one rounding). TL_UNARY_SILU is x*sigmoid(x) through
 * float (the reference's CUDA kernel and CPU float route); TL_UNARY_SILU_CPU_HALF the CPU fp16
 * route as shipped (see tl_silu_f16). sqrt / rsqrt of a value <= 0: the reference's CPU code throws
 * std::domain_error (from inside an OpenMP region, which ends the process); like the reference's
 * CUDA kernels this call cannot see the data without a synchronisation and returns the IEEE
 * result instead (NaN, 0 or inf). */
enum { TL_UNARY_NEG = 0, TL_UNARY_SIN = 1, TL_UNARY_COS = 2, TL_UNARY_EXP = 3, TL_UNARY_LOG = 4, TL_UNARY_ABS = 5,
       TL_UNARY_TANH = 6, TL_UNARY_SILU = 7, TL_UNARY_SQRT = 8, TL_UNARY_RSQRT = 9, TL_UNARY_SILU_CPU_HALF = 10 };
TL_API int tl_unary_f16(tl_half* out, const tl_half* in, size_t n, int op, tl_stream stream);
/* Device::add / sub / mul / div with a tensor or a scalar, and pow with a scalar (Device.hpp:61-70,
 * CPU.cpp:277-340): both operands to float, one operation, one rounding. A zero divisor: the
 * reference's CPU code throws std::invalid_argument("Division by zero."); the scalar form does the
 * same here (TL_ERR_INVALID_ARGUMENT), the tensor form returns the IEEE quotient like the
 * reference's CUDA kernel. pow(0, negative) likewise gives inf instead of throwing. */
enum { TL_BINARY_ADD = 0, TL_BINARY_SUB = 1, TL_BINARY_MUL = 2, TL_BINARY_DIV = 3, TL_BINARY_POW = 4 };
TL_API int tl_binary_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, int op, tl_stream stream);
TL_API int tl_binary_scalar_f16(tl_half* out, const tl_half* a, tl_half scalar, size_t n, int op, tl_stream stream);
/* Device::max / min / sum / mean over consecutive runs of reduce_size elements (Device.hpp:73-76,
 * CPU.cpp:342-402): out[n / reduce_size]. TL_NUMERICS_REFERENCE_ORDER adds sequentially in fp16 like
 * the reference (the mean divides by half(reduce_size)); TL_NUMERICS_FAST adds in fp32 and rounds
 * once. max / min are exact in both (the first of several equal values wins). */
enum { TL_REDUCE_MAX = 0, TL_REDUCE_MIN = 1, TL_REDUCE_SUM = 2, TL_REDUCE_MEAN = 3 };
TL_API int tl_reduce_f16(tl_half* out, const tl_half* in, size_t reduce_size, size_t n, int op, int numerics,
                         tl_stream stream);
/* Device::argmax / argmin (Device.hpp:77-78, CPU.cpp:358-402): int32 index of the first extreme
 * value of every run. want_min = 0: argmax (same result as tl_argmax_f16), 1: argmin. */
TL_API int tl_argreduce_f16(int* out_idx, const tl_half* in, size_t reduce_size, size_t n, int want_min,
                            tl_stream stream);
/* type_cast (CPU.cpp:462-486, CUDA.cu:440-464): into half always through float with one rounding
 * from float (an int32 beyond 2^24 is first rounded to float, as the reference does); half to int
 * truncates toward zero. */
enum { TL_CAST_F16_TO_F32 = 0, TL_CAST_F32_TO_F16 = 1, TL_CAST_F16_TO_I32 = 2, TL_CAST_I32_TO_F16 = 3 };
TL_API int tl_cast(void* out, const void* in, size_t n, int kind, tl_stream stream);

/* ---- fused decode stages (one token, fast numerics) ----------------------------------------
 * Each replaces a run of launches of the reference's decode step; the reference lines are the
 * ones the stage covers. All require 16-byte aligned pointers and K % 8 == 0. */
/* attention_norm + wq|wk|wv GEMVs + rotary embedding + KV-cache write
 * (Transformer.cpp:165, :35-53): x[dim] -> q_out[n_q]; k, v rows written at position `pos` of
 * caches laid out (max_seq, n_q) with n_q = local_heads*head_dim. */
TL_API int tl_rmsnorm_qkv_rope_f16(const tl_half* x, const tl_half* norm_w, float eps, const tl_half* wq,
                            const tl_half* wk, const tl_half* wv, tl_half* q_out, tl_half* k_cache,
                            tl_half* v_cache, int dim, int n_q, int head_dim, int pos,
                            tl_stream stream);
/* per-head attention of one query over positions [0, seq_len) of the caches, read in place
 * (Transformer.cpp:56-109). scratch: float[n_heads*splits*(head_dim+2)], counters:
 * uint32[n_heads] zeroed once by the caller. */
TL_API int tl_attn_decode_f16(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache, tl_half* out,
                       float* scratch, unsigned int* counters, int n_heads, int head_dim, int seq_len,
                       int splits, tl_stream stream);
/* tl_attn_decode_f16 for callers that cannot allocate device memory (inside a stream capture,
 * under a fixed memory budget set by an embedding application, or in a serving loop that bans
 * allocator calls after start-up). No counterpart in the reference, which allocates freely.
 * The scratch and the counters live in a fixed array inside the library image (about 0.5 MB of
 * device memory per GPU that loads the library, held until exit), so the call performs no
 * cudaMalloc / cudaFree and needs no buffers beyond its inputs and output.
 * Limits: n_heads <= 128, head_dim <= 256, n_heads*splits*(head_dim+2) <= 131072; larger requests are rejected
 * with TL_ERR_INVALID_ARGUMENT (use tl_attn_decode_f16 with caller-owned scratch instead).
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress); make
 * that first call before starting any stream capture. All calls share the one array: the entry
 * point clears the counters it needs on `stream` before launching, but two calls that overlap
 * on the GPU (different streams, no ordering between them) race on it. */
TL_API int tl_attn_decode_f16_noalloc(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache,
                                      tl_half* out, int n_heads, int head_dim, int seq_len, int splits,
                                      tl_stream stream);
/* causal attention of T query rows at positions start_pos .. start_pos+T-1 over positions
 * [0, start_pos+T) of the caches, in one kernel (Transformer.cpp:56-109 for T > 1: per-head
 * matmul, ScalarDiv, mask, softmax, per-head matmul). q, out: (T, n_heads*head_dim); caches:
 * (max_seq, n_heads*head_dim), read in place. head_dim must be 128; other head sizes return
 * TL_ERR_UNSUPPORTED (the caller composes tl_matmul_batched_f16 and tl_softmax_f16 instead, as
 * the model path does). */
TL_API int tl_attn_prefill_f16(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache, tl_half* out,
                        int T, int start_pos, int n_heads, int head_dim, tl_stream stream);
/* y[n] = residual[n] + sum_k x[k] W[n,k]  (wo / w2 GEMV + EwiseAdd, Transformer.cpp:111+:169,
 * :143+:175). y may alias residual. */
TL_API int tl_gemv_residual_f16(const tl_half* x, const tl_half* W, const tl_half* residual, tl_half* y,
                         int N, int K, tl_stream stream);
/* ffn_norm + w1|w3 GEMVs + SiLU(gate)*up (Transformer.cpp:171, :136-141): x[dim] -> out[hidden]. */
TL_API int tl_rmsnorm_gateup_swiglu_f16(const tl_half* x, const tl_half* norm_w, float eps, const tl_half* w1,
                                 const tl_half* w3, tl_half* out, int hidden, int dim,
                                 tl_stream stream);

/* ---- Llama2 model (model/llama2_7b) -------------------------------------------------------- */
typedef struct tl_llama2_config {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, max_seq_len; /* main.cpp:26-34 */
    int numerics;           /* TL_NUMERICS_* */
    int silu_via_float;     /* 1: SiLU as on the reference's CUDA path; 0: its CPU fp16 route */
    int tp_rank, tp_world;  /* tensor-parallel shard of this process; 0,1 = single GPU */
    int one_kernel_decode;  /* 0: decode step = CUDA graph of fused kernels chained by programmatic
                               dependent launch (default). 1: single GPU only, the whole step as
                               one persistent cooperative kernel with grid barriers. */
} tl_llama2_config;

typedef struct tl_llama2 tl_llama2;

/* Transformer<half>::Transformer (model/llama2_7b/src/Transformer.cpp:186-202): allocates
 * weights, KV caches (1,max_seq,n_heads,head_dim) per layer and activation buffers. */
TL_API int tl_llama2_create(const tl_llama2_config* cfg, tl_llama2** out);
TL_API int tl_llama2_destroy(tl_llama2* m);
/* read_weights (model/llama2_7b/src/main.cpp:36-190) from a host copy of the checkpoint payload
 * (everything after the 28-byte header), or from a file including the header. With tp_world>1
 * each rank keeps its slice: wq/wk/wv/w1/w3 by output rows, wo/w2 by input columns. */
TL_API int tl_llama2_load_payload_host(tl_llama2* m, const tl_half* payload_host, int shared_classifier);
TL_API int tl_llama2_load_file(tl_llama2* m, const char* path);
/* Fill every weight with a seeded N(0, std^2) pattern generated on the device (norm weights = 1);
 * for throughput runs at sizes where a host checkpoint is impractical. */
TL_API int tl_llama2_init_random(tl_llama2* m, uint64_t seed, float std);
/* Transformer<half>::forward (Transformer.cpp:264-299): tokens_host[T] at start_pos.
 * logits_host (optional) receives (T, vocab) fp16 for all positions like the reference returns;
 * last_logits_host (optional) only the final position. Synchronises, and returns TL_ERR_TIMEOUT
 * instead of results if a kernel of the pass gave up on a bounded wait (see tl_device_status). */
TL_API int tl_llama2_forward(tl_llama2* m, const int* tokens_host, int T, int start_pos,
                      tl_half* logits_host, tl_half* last_logits_host);
/* Llama2<half>::generate (model/llama2_7b/src/llama2.cpp:15-101): prefill the prompt, then greedy
 * decode. Every step moves the sampled id device->host and back like the reference does (the device
 * status word travels with it: a timed-out wait ends the call with TL_ERR_TIMEOUT). Stops
 * early on id 1 or 2 only if stop_on_eos != 0. Returns the number of ids written to out_tokens,
 * and wall-clock seconds of the two phases as the reference prints them. */
TL_API int tl_llama2_generate(tl_llama2* m, const int* prompt_host, int n_prompt, int max_new,
                       int stop_on_eos, int* out_tokens_host, int* n_out, double* prefill_seconds,
                       double* decode_seconds);
/* The same, continuing a conversation: the prompt tokens occupy positions start_pos .. and attend
 * to everything already in the KV cache below start_pos (the reference's multi-turn chat keeps a
 * running total_len this way, llama2.cpp:13, :51-52). tl_llama2_generate is start_pos = 0. */
TL_API int tl_llama2_generate_at(tl_llama2* m, int start_pos, const int* prompt_host, int n_prompt, int max_new,
                          int stop_on_eos, int* out_tokens_host, int* n_out, double* prefill_seconds,
                          double* decode_seconds);
/* Device-resident greedy decode: `steps` tokens starting from the id in the model's device-side
 * token slot (left there by a previous forward/generate/decode call), one CUDA-graph replay per
 * token, no host round trip. out_tokens_host (optional) is filled after the last step. Runs on
 * `stream` and synchronises it only when out_tokens_host != NULL; it then also reads the device
 * status word and returns TL_ERR_TIMEOUT if a wait ran out (without out_tokens_host the caller
 * checks tl_device_status itself after its own synchronisation). */
TL_API int tl_llama2_decode_device(tl_llama2* m, int start_pos, int steps, int* out_tokens_host,
                            tl_stream stream);
/* position bookkeeping and introspection */
TL_API int tl_llama2_set_next_token(tl_llama2* m, int token);
TL_API int tl_llama2_kernel_launches(tl_llama2* m, long long* launches); /* kernels enqueued so far */
TL_API int tl_llama2_weight_bytes(tl_llama2* m, long long* bytes);       /* on this rank */
/* Tracing aid (the reference only has wall-clock prints, llama2.cpp:35-99): run ONE decode step
 * at start_pos (token = the id in the device slot) and return device timestamps (ns, %globaltimer)
 * per GEMV phase: stamps_host[phase][3] = {the phase's first instruction, activation vector staged
 * (under tensor parallelism: the exchanged partial sums have arrived and are added), phase done}.
 * Default decode path (graph of kernels): the step runs as plain launches, CTA 0 of every kernel
 * stamps; phases in launch order are qkv, wo, gate/up, w2 per layer, then the classifier
 * (4 * n_layers + 1; attention is the gap between a qkv and the following wo). one_kernel_decode:
 * CTA `cta` stamps qkv, attention, wo, gate/up, w2 per layer, then the classifier. Every rank of a
 * tensor-parallel group must call it together. capacity = entries available. */
TL_API int tl_llama2_decode_profile(tl_llama2* m, int start_pos, int cta, unsigned long long* stamps_host,
                                    int capacity, int* n_phases);
/* Device pointer and local shape of a weight tensor: name in {"tok_embeddings", "attention_norm",
 * "wq", "wk", "wv", "wo", "ffn_norm", "w1", "w2", "w3", "norm", "output"} (the member names of
 * Transformer / TransformerBlock, Transformer.hpp:36-92); layer ignored for the model-level ones. */
TL_API int tl_llama2_tensor(tl_llama2* m, const char* name, int layer, void** dptr, int* rows, int* cols);

/* ---- tensor parallelism (no counterpart in the reference, which is single-GPU) ---------------
 * One process per GPU. Rank 0 creates an id, every rank passes the same 128 bytes to tl_tp_init
 * (any out-of-band channel carries them), then attaches the group to its model shard, which was
 * created with the same tp_rank / tp_world. wq/wk/wv/w1/w3 and the classifier are split by output
 * rows, wo/w2 by input columns; the forward sums the partial results of wo and w2 over NVLink
 * (NCCL allreduce; decode partials travel as fp32 and are rounded once after the sum). */
TL_API int tl_tp_unique_id(void* out128, int nbytes);
TL_API int tl_tp_init(const void* unique_id, int nbytes, int rank, int world);
TL_API int tl_tp_attach(tl_llama2* m);
TL_API int tl_tp_allreduce_f32(float* buf, size_t n, tl_stream stream);
TL_API int tl_tp_destroy(void);
/* Fused exchange for the decode step: instead of an NCCL allreduce after wo and w2, the GEMV
 * kernels store their fp32 partial sums into a receive region in every rank's memory (peer
 * stores over NVLink) and the next GEMV's prologue sums them in rank order; the classifier
 * slices travel the same way. Every 8-byte word carries its payload and the epoch of the step, so
 * validity needs no separate flag or fence. Needs an even vocabulary slice per rank. Set-up: every rank exports a 64-byte handle of its region, the
 * handles are gathered out of band (rank order, world*64 bytes), every rank opens them; all
 * ranks must pass a host barrier before the first decode step and before closing. Device-side
 * waits are bounded: a consumer retries for roughly two seconds (2^21 polls of its slots), then records
 * TL_ERR_TIMEOUT in the device status word and carries on with what it has; the model calls that
 * synchronise (forward, generate, decode_device with out_tokens_host) turn that word into their
 * return code. Ranks whose launches may drift apart by more than that (first-call graph
 * instantiation, an allocation on one rank) should pass a host barrier first. */
TL_API int tl_tp_exchange_export(tl_llama2* m, void* handle64, int nbytes);
TL_API int tl_tp_exchange_open(tl_llama2* m, const void* handles, int world);
TL_API int tl_tp_exchange_close(tl_llama2* m);
/* Self-test of the bounded device-side wait (no counterpart in the reference, whose kernels never
 * wait on anything): launches one consumer GEMV whose tensor-parallel input comes from a local
 * two-rank receive region that nobody ever posts to, with the wait limited to max_polls polls
 * (1 .. 2^20). The kernel must return by itself; the call synchronises `stream` and returns
 * TL_OK, after which tl_device_status() reports TL_ERR_TIMEOUT once and the library stays usable.
 * Nothing faults or traps. Allocates and frees its own few KB. */
TL_API int tl_selftest_unposted_exchange(int max_polls, tl_stream stream);
/* Self-test of the tensor-parallel prefill exchange on ONE GPU, the ranks emulated by one stream over all
 * ranks' data (no kernel waits for another launch): the K-split matmul in signalling mode computes
 * P = A[M,K] B[dim,K]^T and raises its flags as source rank `owner`... every other source's flags are
 * pre-set and every source's partial points at the same P, so the owner-side kernel of rank `owner`
 * (rows [owner M/world, (owner+1) M/world)) must produce residual_out = residual + half(world x P) and
 * xn = RMSNorm(residual_out) * norm_w in each of the `world` destination copies xn_out[d][M][dim] (rows of
 * other owners stay untouched). All pointers are device memory; residual / residual_out hold the owner's
 * M / world rows. M must be a multiple of 128 x world, world 2, 4 or 8. Synchronises `stream`. */
TL_API int tl_selftest_tp_prefill_exchange(const tl_half* A, const tl_half* B, const tl_half* residual,
                                           const tl_half* norm_w, tl_half* residual_out, tl_half* xn_out,
                                           int M, int dim, int K, int world, int owner, float eps,
                                           tl_stream stream);
/* Host-only: the block of a [rows, cols] checkpoint tensor that rank `rank` of `world` keeps.
 * kind 0 = replicated, 1 = split by rows, 2 = split by columns. */
TL_API int tl_tp_shard(int kind, int rows, int cols, int rank, int world, int* row0, int* nrows,
                       int* col0, int* ncols);

#ifdef __cplusplus
}
#endif
#endif /* TENSORLIB_B200_H */
