/*
 * tfp8b -- C ABI of the B200 (sm_100a) FP8Linear kernels.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the given CUDA
 * stream of the CURRENT device and returns immediately: 0 on success, a negative TFP8B_ERR_*
 * code otherwise (tfp8b_last_error_string() holds the detail for the calling thread). Unless
 * its comment says otherwise an entry point never allocates or frees device memory, never
 * synchronises and keeps no mutable global state, so the codec, prep, GEMV and GEMM calls may be
 * captured in a CUDA graph and issued from several threads or streams at once. All buffers are owned by the caller and must
 * stay alive until the stream has passed the call.
 *
 * Each declaration names the interface of the reference project (tfp8, Turing NVRTC kernels
 * launched with cuLaunchKernel from tfp8/_ext.py) that it replaces, as file:line inside that
 * project.
 *
 * Layouts (all row-major, contiguous):
 *   codes  uint8  [N, K]      FP8 bit patterns, E4M3FN or E5M2
 *   scale  f32    [N, K/G]    or uint8 [N, K/G] (UE8M0: value 2^(b-127), 255 = NaN); G == K means
 *                             one scale per output channel
 *   bias   f32    [N]         or NULL
 *   x      f16 | bf16 | f32 [M, K]
 *   y      f16 | bf16 | f32 [M, N]
 */
#ifndef TFP8B_H_
#define TFP8B_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TFP8B_VERSION 100

#if defined(__GNUC__)
#define TFP8B_API __attribute__((visibility("default")))
#else
#define TFP8B_API
#endif

/* element types of activations / outputs; the numbering is the reference's DT_F16/DT_BF16/DT_F32
 * (tfp8/csrc/tfp8_kernels.cu:127) */
enum { TFP8B_F16 = 0, TFP8B_BF16 = 1, TFP8B_F32 = 2 };
/* FP8 formats; the numbering is FMT_ID (tfp8/_ext.py:41) */
enum { TFP8B_E4M3FN = 0, TFP8B_E5M2 = 1 };
/* weight-scale storage */
enum { TFP8B_SCALE_F32 = 0, TFP8B_SCALE_UE8M0 = 1 };
/* what a NaN input encodes to: CAST = sign|0x7F in both formats (what quantize_weight's
 * clamp-then-cast produces, tfp8/quantize.py:33-35); CANONICAL = 0x7F (E4M3FN) / 0x7E (E5M2)
 * without sign (tfp8/formats.py:93-95) */
enum { TFP8B_NAN_CAST = 0, TFP8B_NAN_CANONICAL = 1 };

enum {
    TFP8B_OK = 0,
    TFP8B_ERR_INVALID = -1,     /* null pointer, bad enum, negative size, misaligned pointer */
    TFP8B_ERR_UNSUPPORTED = -2, /* shape outside what the kernels serve (K % 32, G % 32, ...) */
    TFP8B_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed */
    TFP8B_ERR_DEVICE = -4       /* a kernel reported a problem in the device status word (see tfp8b_device_status) */
};

/* bits of the device status word */
enum {
    TFP8B_STATUS_GEMV_WAIT = 1, /* a decode-GEMV CTA gave up on a bounded wait: its outputs are incomplete */
    TFP8B_STATUS_GEMM_WAIT = 2, /* the same for the tile GEMM */
    TFP8B_STATUS_GLUE_WAIT = 4, /* tfp8b_allreduce_add_rmsnorm: a peer never raised its flag; the rows were set to NaN */
    TFP8B_STATUS_GLUE_POS = 8   /* tfp8b_rope_kv_store: a position outside [0, max_seq) was skipped */
};

typedef void* tfp8b_stream_t; /* a cudaStream_t */

/* Library version (TFP8B_VERSION at build time). No reference counterpart. */
TFP8B_API int tfp8b_version(void);

/* Text of the last error on the calling thread ("" if none). Replaces the RuntimeError text built
 * from cuLaunchKernel's return code (tfp8/_ext.py:156-157, 215-216). */
TFP8B_API const char* tfp8b_last_error_string(void);

/* Reads and clears the device-side status word of the current device (TFP8B_STATUS_* bits): 0 = no
 * kernel has given up on a bounded wait or skipped an out-of-range position since the last call.
 * SYNCHRONISES the stream. out_status may be NULL. Returns TFP8B_ERR_DEVICE when the word was
 * non-zero. No reference counterpart (its kernels have no waits). */
TFP8B_API int tfp8b_device_status(unsigned int* out_status, tfp8b_stream_t stream);

/* codes[i] = FP8(x[i]): round to nearest even, saturate to +-max finite, never inf.
 * Replaces the device encoder m_enc16_f16/f32 + enc_e4m3 (tests/bench_transcode.py:206-225,
 * 319-343) and the elementwise part of quantize_weight (tfp8/quantize.py:33-35). */
TFP8B_API int tfp8b_encode(const void* x, int x_dtype, uint8_t* codes, int64_t n, int fmt, int nan_mode,
                 tfp8b_stream_t stream);

/* out[i] = value of codes[i] in out_dtype (exact; NaN, inf and -0 kept).
 * Replaces m_dec16_* (tests/bench_transcode.py:228-317) / lut(fmt)[codes] (tfp8/formats.py:63). */
TFP8B_API int tfp8b_decode(const uint8_t* codes, void* out, int out_dtype, int64_t n, int fmt,
                 tfp8b_stream_t stream);

/* One-pass weight quantizer: per (row, K-group) amax -> scale -> codes.
 *   s = max(amax / fmax, FLT_MIN); pow2 != 0: s = 2^ceil(log2 s); s = 1 where amax == 0;
 *   codes = FP8(clamp(w / s, +-fmax)).  scale_kind UE8M0 needs pow2 != 0.
 * Replaces quantize_weight (tfp8/quantize.py:15-36). K % G == 0, G % 16 == 0. */
TFP8B_API int tfp8b_quantize(const void* w, int w_dtype, uint8_t* codes, void* scale, int scale_kind,
                   int N, int K, int G, int fmt, int pow2, tfp8b_stream_t stream);

/* out[n,k] = out_dtype(decode(codes[n,k]) * scale[n, k/G]); out_dtype f16 (the reference's
 * workspace type), bf16 or f32. Replaces tfp8_dequant_f16 / dequant_into
 * (tfp8/csrc/tfp8_kernels.cu:435-456, tfp8/_ext.py:305-315). K % 16 == 0, G % 16 == 0. */
TFP8B_API int tfp8b_dequant(const uint8_t* codes, const void* scale, int scale_kind, void* out,
                  int out_dtype, int N, int K, int G, int fmt, tfp8b_stream_t stream);

/* Activation rows -> fp16 with an exact power-of-two row scale: e = ceil(log2 amax) - 8
 * (0 for an all-zero row), x16 = fp16(x / 2^e), xs = 2^e. Replaces tfp8_prep_{f16,bf16,f32} /
 * prepare_activations (tfp8/csrc/tfp8_kernels.cu:513-539, tfp8/_ext.py:220-227). K % 8 == 0. */
TFP8B_API int tfp8b_prep(const void* x, int x_dtype, void* x16, float* xs, int M, int K,
               tfp8b_stream_t stream);

/* Decode GEMV, 1 <= M <= 8:  y[m,n] = sum_g scale[n,g] * sum_{k in g} x[m,k]*dec(codes[n,k]) + bias[n]
 * with x consumed in its own dtype and FP32 accumulation. Replaces the 27 tfp8_gemv_in_*_m*_*
 * kernels and their launcher (tfp8/csrc/tfp8_kernels.cu:171-269, 414-425; tfp8/_ext.py:163-217,
 * 230-250). K % 32 == 0, G % 32 == 0, x / codes 16-byte aligned. */
TFP8B_API int tfp8b_gemv(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
               const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
               tfp8b_stream_t stream);

/* Ordering contract of the decode GEMVs (tfp8b_gemv, tfp8b_gemv_ex, tfp8b_gemv_normed,
 * tfp8b_gemv_gated, tfp8b_gemv_plan_run). They are launched with programmatic dependent launch:
 * the kernel may start while the kernel BEFORE it in the stream is still running, and reads
 *   codes, scale, bias   at once, without waiting for that kernel;
 *   x (and the inputs of the normed / gated forms), y   only after that kernel has completed.
 * So the kernel that immediately precedes a GEMV in its stream must not WRITE that GEMV's codes,
 * scale or bias (weights are normally written once, long before). A caller that does update
 * weights in the kernel just before -- a requantize, a LoRA merge -- passes TFP8B_GEMV_NO_PDL,
 * which makes the call an ordinary stream-ordered launch, or puts any other kernel in between.
 *
 * tfp8b_gemv with flags.
 * TFP8B_GEMV_INDEPENDENT_IO: the caller vouches that x and y are neither written nor read by the
 * kernel that precedes this call in the stream -- as for the K and V projections that follow the
 * Q projection of the same activations, or the layers of a sweep. The call then runs
 * concurrently with that kernel (no wait in front of the activations); it still never completes
 * before its predecessor, so later work in the stream sees both finished.
 * TFP8B_GEMV_NO_PDL: plain launch, nothing is read before the predecessor has completed.
 * No reference counterpart. */
#define TFP8B_GEMV_INDEPENDENT_IO 1u
#define TFP8B_GEMV_NO_PDL 2u
TFP8B_API int tfp8b_gemv_ex(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                  const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                  unsigned int flags, tfp8b_stream_t stream);

/* A decode GEMV prepared once per layer: the tensor map of the weight stream, the shared-memory
 * plan and the kernel choice are worked out when the plan is made, so a call costs one kernel
 * launch and nothing else (tfp8b_gemv builds a tensor map per call). Replaces the reference's
 * prepared launch, GemvLaunch (tfp8/_ext.py:163-217), which binds every argument but x, y and M.
 *   create   binds codes / scale / bias / shape / types on the CURRENT device for 1 <= max_M <= 8
 *            rows; *plan receives an opaque handle (host memory only, no device allocation).
 *   run      y[0:M] = x[0:M] W^T (+ bias) for 1 <= M <= max_M; x, y as in tfp8b_gemv; flags as in
 *            tfp8b_gemv_ex. The bound buffers must still be alive and unchanged in address.
 *   destroy  frees the handle (NULL is allowed).
 * A plan may be used from several threads and streams at once. */
typedef struct tfp8b_gemv_plan tfp8b_gemv_plan;
TFP8B_API int tfp8b_gemv_plan_create(tfp8b_gemv_plan** plan, int x_dtype, const uint8_t* codes, const void* scale,
                  int scale_kind, const float* bias, int y_dtype, int max_M, int N, int K, int G, int fmt);
TFP8B_API int tfp8b_gemv_plan_run(const tfp8b_gemv_plan* plan, const void* x, void* y, int M, unsigned int flags,
                  tfp8b_stream_t stream);
TFP8B_API void tfp8b_gemv_plan_destroy(tfp8b_gemv_plan* plan);

/* Tile GEMM for any M >= 1 on prepared activations (tfp8b_prep):
 *   y[m,n] = xs[m] * sum_k x16[m,k] * dec(codes[n,k]) * scale[n,k/G] + bias[n]
 * FP8 tiles are decoded to fp16 in shared memory (group scales folded in as scale/rowmax),
 * multiplied by tcgen05.mma with FP32 accumulators in tensor memory. Replaces tfp8_gemm_* /
 * gemm_prepared and the chunked dequant+cuBLAS+epilogue path (tfp8/csrc/tfp8_kernels.cu:288-411,
 * 428-430; tfp8/_ext.py:259-275; tfp8/linear.py:107-128). K % 32 == 0, G % 32 == 0,
 * x16 / codes 16-byte aligned. Builds two tensor maps on the host per call (no allocation). */
TFP8B_API int tfp8b_gemm(const void* x16, const float* xs, const uint8_t* codes, const void* scale,
               int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K, int G,
               int fmt, tfp8b_stream_t stream);

/* ---- W8A8: FP8 activations x FP8 weights (the reference project's second native kernel,
 * fp8_gemm_kernel.cu, and its binding fp8_cuda.py) ----
 *
 * tfp8b_gemm_w8a8:  y[m,n] = sum_k dec(a[m,k]) * dec(w[n,k]) * (scales) + bias[n], FP32 accumulation.
 *   a_codes u8 [M, K], w_codes u8 [N, K] (both row-major, K contiguous), E4M3FN or E5M2 each.
 *   scale_mode TFP8B_W8A8_BLOCK32: one scale per row and 32-wide block of K, applied to each block's
 *       partial product (fp8_gemm_kernel.cu:86-103, SCALE_BLOCK_K). With scale_kind UE8M0 the scales
 *       are exponent bytes in the PACKED layout below and the tensor cores apply them
 *       (tcgen05.mma.kind::mxf8f6f4.block_scale); with scale_kind F32 they are float32 [rows, K/32]
 *       row-major and every block goes through an FP32 register accumulation (correct, slow).
 *   scale_mode TFP8B_W8A8_ROWCOL: a_scale [M], w_scale [N] (float32 or UE8M0 bytes), applied once
 *       in the epilogue (fp8_gemm_kernel.cu:113-120, SCALE_ROW_COL).
 *   Replaces the four kernels gemm_{block,rowcol}_{fp32,ue8m0} (fp8_gemm_kernel.cu:123-126) and
 *   their launch (fp8_cuda.py:94-138). The reference stores the weight as [K, N] with scales
 *   [K/32, N]; here both operands are K-major, the layout FP8Linear keeps (transpose once at load).
 *   K % 128 == 0; codes and scales 16-byte aligned. y f32 (the reference's output type), f16 or bf16.
 * PACKED scale layout: for every 128 rows x 128 K one 512-byte chunk, the byte of (row r, block b) at
 *   (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4), chunks ordered [r / 128][b / 4]; rows and blocks
 *   beyond the tensor hold 127 (= 1.0). tfp8b_mx_packed_scale_bytes gives the buffer size,
 *   tfp8b_mx_pack_scales converts row-major UE8M0 bytes [rows, K/32] (weights: once at load).
 * tfp8b_quantize_k: rows -> FP8 codes + one scale per 32-wide block of K, the reference's dynamic
 *   activation quantizer quantize_k (fp8_cuda.py:74-91): s = max(amax / fmax, 1e-12); with ue8m0
 *   e = clamp(ceil(log2 s), -127, 127), s = 2^e, byte e + 127; codes = FP8(clamp(x / s)). scale:
 *   float32 [rows, K/32], or UE8M0 bytes row-major (packed == 0) or in the packed layout. */
enum { TFP8B_W8A8_BLOCK32 = 0, TFP8B_W8A8_ROWCOL = 1 };
TFP8B_API int tfp8b_gemm_w8a8(const uint8_t* a_codes, const void* a_scale, int a_fmt, const uint8_t* w_codes, const void* w_scale,
                  int w_fmt, int scale_mode, int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K,
                  tfp8b_stream_t stream);
TFP8B_API long long tfp8b_mx_packed_scale_bytes(int rows, int K);
TFP8B_API int tfp8b_mx_pack_scales(const uint8_t* scale_rowmajor, uint8_t* packed, int rows, int K, tfp8b_stream_t stream);
TFP8B_API int tfp8b_quantize_k(const void* x, int x_dtype, uint8_t* codes, void* scale, int rows, int K, int fmt, int ue8m0,
                  int packed, tfp8b_stream_t stream);

/* The whole linear layer for any M >= 1 in one call that allocates nothing:
 *   y = x @ dequant(codes).T + bias   (activation prep, then the tile GEMM)
 * This entry point has no counterpart in the reference. It exists for callers that cannot obtain
 * device memory at the moment they need the layer: serving loops in which an allocation would
 * stall every other stream of the device, processes whose device-memory budget was fixed at
 * start-up, and hosts that bind this library through a foreign-function interface without a
 * CUDA allocator of their own. The prepared activations, which tfp8b_prep / tfp8b_gemm keep in caller memory,
 * live here in an 8 MiB array inside the library (present on every GPU that loads it, until the
 * process ends).
 *   Limits: M <= 8192 and M * K <= 4 Mi values per call; larger calls are refused with
 *           TFP8B_ERR_UNSUPPORTED and a message that names the limit.
 *   First call on a device: looks up the array's device address (a host-side query, no
 *           allocation); make that call before any stream capture begins.
 *   The array is shared by every call and keeps what the last call wrote; each call rewrites all
 *           of what it reads. Two calls that overlap on the GPU (different streams) race on it:
 *           issue them on one stream, or order them with events.
 * x: f16 | bf16 | f32 [M, K]; the other arguments as for tfp8b_gemm. */
TFP8B_API int tfp8b_linear_static(const void* x, int x_dtype, const uint8_t* codes, const void* scale,
                  int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K, int G,
                  int fmt, tfp8b_stream_t stream);

/* y[m, 0:n] = y_dtype(acc[m, 0:n] * xs[m] + bias[0:n]) into a column window of a wider output
 * (row pitch ldy elements). Replaces tfp8_epilogue_* / epilogue_into
 * (tfp8/csrc/tfp8_kernels.cu:478-503, tfp8/_ext.py:282-302). */
TFP8B_API int tfp8b_epilogue(const float* acc, const float* xs, const float* bias, void* y, int y_dtype,
                   int M, int n, int ldy, tfp8b_stream_t stream);

/* Decode-step helpers around the FP8Linear layers of a Llama-style block (the reference's demo,
 * tfp8/examples/demo_llm.py:64-87, does this work with eager torch kernels).
 * tfp8b_rope_kv_store: rotary embedding (rotate-half pairs i, i + hd/2) of the Q and K heads of a
 * fused projection output qkv [B, T, H + 2*KV, hd]; Q goes to q_out [B, H, T, hd], K and V into the
 * static caches [B, KV, max_seq, hd] at positions pos[t] (int64, on the device). cos / sin are
 * f32 [max_seq, hd/2]. dtype f16 or bf16. A token whose position lies outside [0, max_seq) is
 * skipped (no table read, no store, its q_out rows are left as they were) and
 * TFP8B_STATUS_GLUE_POS is raised in the device status word. */
TFP8B_API int tfp8b_rope_kv_store(const void* qkv, int dtype, const long long* pos, const float* cosv,
                  const float* sinv, void* q_out, void* k_cache, void* v_cache, int B, int T, int H,
                  int KV, int hd, int max_seq, tfp8b_stream_t stream);

/* out[r, 0:F] = silu(gate_up[r, 0:F]) * gate_up[r, F:2F]; f16 or bf16, F % 8 == 0 (reference:
 * tfp8/examples/demo_llm.py:86-87). */
TFP8B_API int tfp8b_silu_mul(const void* gate_up, void* out, int dtype, long long rows, int F,
                  tfp8b_stream_t stream);

/* Decode GEMVs that compute their activations instead of reading them, which takes one kernel out
 * of the dependent chain of a decode step each (every CTA recomputes the M <= 8 rows from L2):
 *   tfp8b_gemv_normed  x = RMSNorm(residual + delta) * norm_weight (delta may be NULL), y = x W^T;
 *                      the updated residual is also stored to residual_out (NULL to skip), which
 *                      must not be `residual` itself when delta is given;
 *   tfp8b_gemv_gated   x = silu(gate_up[:, 0:K]) * gate_up[:, K:2K] for a fused gate/up output
 *                      [M, 2K], y = x W^T.
 * f16 / bf16 activations, rows short enough to stay in shared memory (M * K * 2 <= 96 KB); the
 * other arguments as tfp8b_gemv. (Reference: RMSNorm, residual adds and SwiGLU of
 * tfp8/examples/demo_llm.py:30-39, 86-87, 98-101 around its FP8Linear calls.) */
TFP8B_API int tfp8b_gemv_normed(void* residual_out, const void* residual, const void* delta, const void* norm_weight,
                  float eps, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                  const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                  tfp8b_stream_t stream);
TFP8B_API int tfp8b_gemv_gated(const void* gate_up, int x_dtype, const uint8_t* codes, const void* scale,
                  int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K, int G,
                  int fmt, tfp8b_stream_t stream);

/* tfp8b_gemm whose N output columns land at columns [col0, col0 + N) of wider outputs (row pitch
 * ldy elements), in n_dst buffers at once (1..8; y_dst is a HOST array of device pointers). With
 * the buffers of every GPU of a tensor-parallel group (peer-mapped memory: CUDA IPC, symmetric
 * memory) a column-sharded layer writes its shard straight into every rank's full output: the
 * all-gather happens in the GEMM's epilogue, as plain stores over NVLink, overlapped with the
 * main loop of the next tiles. The caller orders the ranks afterwards (a barrier) before anyone
 * reads. No counterpart in the reference (single GPU). */
TFP8B_API int tfp8b_gemm_scatter(const void* x16, const float* xs, const uint8_t* codes, const void* scale,
                  int scale_kind, const float* bias, void* const* y_dst, int n_dst, long long ldy,
                  long long col0, int y_dtype, int M, int N, int K, int G, int fmt, tfp8b_stream_t stream);

/* tfp8b_gemm with an FP32 workspace of at least M * N floats. With one activation tile (M <= 256)
 * and few 128-row weight tiles of a long K, the call cuts every tile into units along K that
 * run on different SMs, adds their partial results into the workspace (atomic adds: the last
 * bits of a result can differ from run to run) and applies activation scale and bias in a final
 * pass; whether and how far it splits follows a cost model, and TFP8B_GEMM_SPLITK=0 in the
 * environment turns it off. With at least one tile per SM but a badly filled last round (224
 * tiles on 148 SMs) it splits by spans instead: the k-blocks of all tiles, tile after tile, are
 * dealt out in equal contiguous spans, one per SM; a tile then gets its sum from at most two
 * CTAs, so this form gives the same bits on every run (TFP8B_GEMM_SPANS=0 turns it off).
 * Without a split the workspace is not touched and the result is tfp8b_gemm's, bit for bit.
 * No counterpart in the reference. */
TFP8B_API int tfp8b_gemm_splitk(const void* x16, const float* xs, const uint8_t* codes, const void* scale,
                  int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K, int G,
                  int fmt, float* workspace, long long workspace_floats, tfp8b_stream_t stream);

/* x[r, :] += delta[r, :] (delta may be NULL), then out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps)
 * * weight: the residual update and the RMSNorm that follows it in a decoder block, one launch
 * (reference: RMSNorm and the residual adds of tfp8/examples/demo_llm.py:30-39, 98-101; same
 * arithmetic: FP32 inside, one rounding to the activation type). f16 or bf16, dim % 8 == 0,
 * all buffers 16-byte aligned; x is updated in place. */
TFP8B_API int tfp8b_add_rmsnorm(void* x, const void* delta, const void* weight, void* out, int dtype,
                  long long rows, int dim, float eps, tfp8b_stream_t stream);

/* tfp8b_add_rmsnorm whose addend is the SUM over the ranks of a tensor-parallel group of FP32 partial
 * results [rows, dim] (the output of a row-parallel projection): the all-reduce, the residual
 * update and the RMSNorm in one launch, for the few rows of a decode step. Each rank pushes its
 * partial rows into every peer's receive area with plain peer stores, raises a per-row flag, waits
 * (bounded) for the peers' flags and adds the partials in rank order, so every rank computes the
 * same bits. recv[r] / flags[r] (HOST arrays of `world` device pointers, peer-mapped memory) are
 * rank r's receive area, 2 * world * max_rows * dim floats, and flag array, 2 * world * max_rows
 * uint32, both zeroed once before the first call; state is two zeroed uint32 of local device
 * memory (the call sequence number lives there, which keeps the call replayable from a CUDA
 * graph). Every rank issues the same calls in the same order; world <= 8, dim <= 4096.
 * No counterpart in the reference (single GPU). */
TFP8B_API int tfp8b_allreduce_add_rmsnorm(void* x, const float* partial, const void* weight, void* out, int dtype,
                  int rows, int dim, float eps, float* const* recv, unsigned int* const* flags,
                  unsigned int* state, int rank, int world, int max_rows, tfp8b_stream_t stream);

/* Sets how long (SM clock cycles, > 0) a CTA of tfp8b_allreduce_add_rmsnorm waits for a peer's flag
 * before it gives up, for all later calls of this process; returns the previous limit (2^35 cycles,
 * about 17 seconds, by default; cycles <= 0 only queries). When the wait runs out the kernel does not sum
 * stale data: it sets the row to NaN in x and out, raises TFP8B_STATUS_GLUE_WAIT and returns.
 * No counterpart in the reference. */
TFP8B_API long long tfp8b_allreduce_wait_limit(long long cycles);

/* One-query attention over the static KV cache, grouped-query heads: for every sequence b and head h,
 * out[b, h, :] = softmax(q[b, h, :] . K[b, h / (H/KV), 0:pos+1, :]^T / sqrt(hd)) V[...]. q and out are
 * [B, H, hd]; the caches [B, KV, max_seq, hd]; pos is ONE int64 on the device (the cache position of
 * the current token, already written by tfp8b_rope_kv_store). scratch: at least
 * B * H * ceil(max_seq / 64) * (hd + 2) floats of device memory for the split-KV partial results
 * (one record per head and 64-position chunk of the cache). f16 or bf16, hd = 128. fp16 runs both
 * products on the tensor cores (fp16 operands, FP32 accumulation, the softmax weights as an fp16
 * high + low part; 128 or 256 positions per chunk); bf16 is scalar FP32. (Reference: the torch
 * attention of tfp8/examples/demo_llm.py:64-76.) */
TFP8B_API int tfp8b_attn_decode(const void* q, const void* k_cache, const void* v_cache, const long long* pos,
                  void* out, float* scratch, long long scratch_floats, int dtype, int B, int H, int KV, int hd,
                  int max_seq, tfp8b_stream_t stream);

/* The two calls above over an FP8 KV cache -- the mode the reference's FP8Config reserves and
 * refuses (kv_cache != "fp16": tfp8/config.py:27-28). k_codes / v_codes u8 [B, KV, max_seq, hd],
 * k_scale / v_scale f32 [B, KV, max_seq]: K (after the rotation) and V are rounded to the
 * activation type, as the 16-bit cache holds them, and then quantized per token and KV head the way
 * quantize_weight quantizes a row (tfp8/quantize.py:15-36: scale 2^ceil(log2(amax / fmax)), 1 for
 * an all-zero row; round to nearest even, saturating) -- tfp8b_quantize on the 16-bit cache rows
 * gives the same bytes. The attention decodes the codes to fp16 in registers (exact) and runs both
 * products on the tensor cores with FP32 accumulation: score = (q . codes) * k_scale in FP32, the
 * softmax weights as an fp16 high + low part, the V scales as exact powers of two. hd = 128; fmt
 * E4M3FN or E5M2. k_codes and v_codes 16-byte aligned. Scratch: B * H * ceil(max_seq / 128) * 130
 * floats at least (tfp8b_attn_decode's size is enough). */
TFP8B_API int tfp8b_rope_kv_store_fp8(const void* qkv, int dtype, const long long* pos, const float* cos_table,
                  const float* sin_table, void* q_out, uint8_t* k_codes, float* k_scale, uint8_t* v_codes,
                  float* v_scale, int B, int T, int H, int KV, int hd, int max_seq, int fmt, tfp8b_stream_t stream);
TFP8B_API int tfp8b_attn_decode_fp8(const void* q, const uint8_t* k_codes, const float* k_scale, const uint8_t* v_codes,
                  const float* v_scale, const long long* pos, void* out, float* scratch, long long scratch_floats,
                  int dtype, int B, int H, int KV, int hd, int max_seq, int fmt, tfp8b_stream_t stream);

/* out[r] = argmax over logits[r, 0:n] (row pitch in elements), int64; the lowest index among equal
 * values, NaN counts as largest -- the greedy sampling step of the reference's demo
 * (tfp8/examples/demo_llm.py:149). f16 or bf16. */
TFP8B_API int tfp8b_argmax(const void* logits, int dtype, long long* out, long long rows, long long n,
                  long long row_pitch, tfp8b_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TFP8B_H_ */
