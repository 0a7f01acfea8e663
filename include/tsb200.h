/* tsb200.h - C ABI of the B200 (sm_100a) compressed-decode kernels.
 *
 * This library replaces, for one hot path, what transformer-surgeon executes through
 * PyTorch library calls: LinearCompressed.forward on quantized low-rank factors, a
 * quantized paged KV cache (append + decode attention) and the small decoder ops around
 * them.  The reference project ships no native code and therefore no FFI; each entry
 * point below names the reference Python function whose arithmetic it takes over
 * (paths are relative to the reference project root).
 *
 * Conventions
 *   - every function returns 0 (TSB200_OK) or a negative tsb200_status; it never throws,
 *     never allocates device memory, never synchronises the device; work is enqueued on
 *     the `stream` argument (a cudaStream_t passed as void*; NULL = legacy default stream);
 *   - all pointers are DEVICE pointers unless the name ends in `_host`;
 *   - tensors are dense row-major; "act dtype" is the dtype of activations/bias/outputs;
 *   - scratch memory is supplied by the caller (`workspace`, sized by the matching
 *     `*_workspace_bytes` function);
 *   - the library contains sm_100a code only: on any other device every compute entry
 *     point returns TSB200_ERR_DEVICE (there is no fallback path).
 */
#ifndef TSB200_H
#define TSB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TSB200_OK = 0,
  TSB200_ERR_ARG = -1,         /* null pointer, negative size, misaligned pointer        */
  TSB200_ERR_UNSUPPORTED = -2, /* shape / dtype / format combination not implemented     */
  TSB200_ERR_CUDA = -3,        /* a CUDA runtime call failed (see tsb200_last_cuda_error)*/
  TSB200_ERR_WORKSPACE = -4,   /* workspace too small                                    */
  TSB200_ERR_DEVICE = -5,      /* current device is not compute capability 10.0          */
  TSB200_ERR_TIMEOUT = -6      /* a bounded device-side wait ran out (status word set)   */
} tsb200_status;

typedef enum { TSB200_F32 = 0, TSB200_BF16 = 1 } tsb200_dtype;

/* Weight containers: storage bits per code.  32/16 = unquantized fp32/bf16 weights. */
typedef enum {
  TSB200_W_BIN1 = 1, TSB200_W_INT2 = 2, TSB200_W_INT4 = 4, TSB200_W_INT8 = 8,
  TSB200_W_BF16 = 16, TSB200_W_F32 = 32
} tsb200_wbits;

typedef enum {
  TSB200_KV_INT8 = 0, TSB200_KV_FP8 = 1, TSB200_KV_NVFP4 = 2,
  TSB200_KV_F32 = 3, TSB200_KV_BF16 = 4   /* unquantized pages in the act dtype */
} tsb200_kv_format;

const char* tsb200_strerror(int status);
int tsb200_version(void);
/* cudaError_t of the most recent failing runtime call made by this library (0 if none). */
int tsb200_last_cuda_error(void);
/* TSB200_OK when the CURRENT device can run this library (compute capability 10.0). */
int tsb200_check_device(void);
/* Programmatic dependent launch for the decode-step kernels (linear, rope_append, decode
 * attention, add_rmsnorm, swiglu): when enabled, each launch may start while its predecessor on
 * the stream drains; the kernels order their dependent memory accesses themselves.  Process-wide;
 * returns the previous setting.  Default 0.
 * What a kernel touches before that ordering point is constant data (weights, weight and cache scales, RoPE tables),
 * the lengths and the block table (seq_lens, new_lens, block_table: read by the append and by the decode attention) and,
 * in the FP8 decode attention with one split, pages of the cache STRICTLY OLDER than the one that holds a sequence's
 * newest token.  With this setting on, the launch that directly precedes an append or a decode attention on its stream
 * must therefore not be the one that writes those: advance lengths, remap pages and refresh scales at least two launches
 * ahead (the engine of this package does so at the start of a step), or turn the setting off around such a pair. */
int tsb200_set_pdl(int enabled);

/* ------------------------------------------------------------------------------------
 * Weight quantization, packing, reconstruction
 * Replaces: compression/quantization_methods/vanilla.py:10-24 (_quantize_maxabs),
 *           :27-37 (_quantize_binarize), :5-7 (_dequantize_symmetric) and the write-back
 *           compression/quantization.py:112,126.
 * Arithmetic follows the reference bit for bit: all steps in the parameter dtype
 * (bf16: fp32 op then round-to-nearest-even to bf16 after EVERY op), round-half-even.
 * ---------------------------------------------------------------------------------- */

/* Bytes of one packed row: ceil(cols/64)*64*bits/8 (bits in 1,2,4,8). 0 on bad args. */
size_t tsb200_packed_row_bytes(int64_t cols, int bits);

/* w [rows, cols] (dtype) -> codes int8 [rows, cols], scales fp32 [rows] (values exactly
 * representable in `dtype`; per-tensor mode writes the same scale to every row).
 * precision: 2..8 fixed point, 0 = binary (sign, mean|w|).  workspace: >= 16 bytes. */
int tsb200_quantize_weight(const void* w, int dtype, int64_t rows, int64_t cols,
                           int precision, int per_channel, float eps,
                           int8_t* codes, float* scales,
                           void* workspace, size_t workspace_bytes, void* stream);

/* codes int8 [rows, cols] -> packed [rows, tsb200_packed_row_bytes(cols,bits)].
 * Container: bits=8 one byte per code in column order; bits<8 little-endian 32-bit words
 * of per = 32/bits fields covering `per` consecutive columns, pair-interleaved (field
 * i < per/2 = column 2i of the group, field i >= per/2 = column 2(i-per/2)+1), two's
 * complement fields (bits=1: 1 -> +1, 0 -> -1); rows zero-padded to 64 columns.
 * bits=1 requires codes in {-1,+1}; *zero_flag (device int32, may be NULL) is set to 1
 * when a zero code was met (the caller then repacks with bits=2). */
int tsb200_pack_codes(const int8_t* codes, int64_t rows, int64_t cols, int bits,
                      uint8_t* packed, int32_t* zero_flag, void* stream);

/* packed -> codes int8 [rows, cols]. */
int tsb200_unpack_codes(const uint8_t* packed, int64_t rows, int64_t cols, int bits,
                        int8_t* codes, void* stream);

/* packed + scales -> w_out [rows, cols] (dtype) = RN_dtype(float(code) * scale[row]):
 * the fake-quantized weight the reference stores (quantization.py:126). */
int tsb200_dequantize_weight(const uint8_t* packed, const float* scales, int64_t rows,
                             int64_t cols, int bits, int dtype, void* w_out, void* stream);

/* ------------------------------------------------------------------------------------
 * LinearCompressed.forward
 * Replaces: blocks/linear_compressed.py:81-105
 *   h = x @ V^T        (only when rank > 0;  V = linear_V.weight [rank, in])
 *   y = h @ U^T + bias (U = weight [out, rank] or [out, in])
 * A factor is either unquantized (bits 16/32, pointer to act-dtype matrix, scale NULL)
 * or packed codes (bits 1/2/4/8) with one fp32 scale per row.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  int64_t in_features;
  int64_t out_features;
  int64_t rank;          /* 0 = full rank (no V factor)                                 */
  int32_t act_dtype;     /* tsb200_dtype of x, y, bias and of the rank-r intermediate   */
  int32_t u_bits;        /* tsb200_wbits of U                                            */
  int32_t v_bits;        /* tsb200_wbits of V (ignored when rank == 0)                   */
  int32_t reserved;      /* must be 0                                                    */
  const void* u;         /* [out, K] packed or dense, K = rank ? rank : in_features      */
  const float* u_scale;  /* [out] or NULL for dense                                      */
  const void* v;         /* [rank, in] packed or dense, or NULL                          */
  const float* v_scale;  /* [rank] or NULL                                               */
  const void* bias;      /* [out] act dtype, or NULL                                     */
} tsb200_linear_desc;

/* The first 16640 bytes of the workspace (status word + split-K counters) must be zero-filled
 * ONCE by the caller before its first use; every call leaves them reusable.  Byte 0..3
 * is a status word: non-zero after a kernel gave up on a bounded device-side wait.  One workspace
 * must not be used by two calls that may overlap on the GPU. */
size_t tsb200_linear_workspace_bytes(const tsb200_linear_desc* d, int64_t M);
/* x [M, in] -> y [M, out].  M == 0 is a no-op. */
int tsb200_linear(const tsb200_linear_desc* d, const void* x, void* y, int64_t M,
                  void* workspace, size_t workspace_bytes, void* stream);
/* Same contract; forces the CUDA-core streaming kernel (any M; serves fp32 models and shapes the
 * tensor-core kernel does not take, and is the cross-check of the tensor-core kernel). */
int tsb200_linear_simt(const tsb200_linear_desc* d, const void* x, void* y, int64_t M,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Greedy head: tokens[m] = argmax_n (x . W^T + bias)[m, n] with the logits rounded to the act dtype first, i.e. the
 * token torch.argmax would pick from tsb200_linear's output (the first maximum on ties).
 * Replaces the final layer + argmax of a greedy decode step (export/common.py:167,175 for the blocks path; the
 * lm_head call and the argmax of Hugging Face's greedy search for the HF path).  For a dense bf16 full-rank head with
 * M <= 128 the reduction happens in the GEMM's epilogue (per 128-column tile, then one small kernel): the
 * [M, vocabulary] logits are never written or re-read.  Any other head (packed, low-rank, fp32) computes its logits
 * into the workspace and reduces them.  tokens: device int64 [M].  The first 16640 bytes of the workspace follow the
 * rules of tsb200_linear's workspace. */
size_t tsb200_linear_argmax_workspace_bytes(const tsb200_linear_desc* d, int64_t M);
int tsb200_linear_argmax(const tsb200_linear_desc* d, const void* x, int64_t* tokens, int64_t M,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Gated MLP block: y = down(silu(gate(x)) * up(x)).
 * Replaces: blocks/mlp.py:171-185 (MLPGated.forward: up_proj, gate_proj, activation * up, down_proj)
 * with SiLU as the activation (the Qwen2 / Llama choice).  gate and up map in -> inter, down maps
 * inter -> out; x [M, in] -> y [M, out].  When the layers are packed alike the whole block is one
 * launch; otherwise it is composed from tsb200_linear and tsb200_swiglu.  The workspace must be
 * zero-filled once before its first use and must not serve overlapping calls. */
size_t tsb200_mlp_gated_workspace_bytes(const tsb200_linear_desc* gate, const tsb200_linear_desc* up,
                                        const tsb200_linear_desc* down, int64_t M);
int tsb200_mlp_gated(const tsb200_linear_desc* gate, const tsb200_linear_desc* up,
                     const tsb200_linear_desc* down, const void* x, void* y, int64_t M,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------
 * Quantized paged KV cache
 * The reference's cache is a dense fixed-size row store written at clamp(pos_id)
 * (blocks/mha.py:514-535, :583) or Hugging Face's DynamicLayer.update (torch.cat); the
 * quantized/paged formats here are new behaviour layered on the same call points.
 * Page = 16 tokens.  Pools: uint8 [num_pages, hkv, record_bytes]; record layouts:
 *   K int8  : codes [16][d], then fp32 scale [16]
 *   K fp8   : codes [16][d]                         (e4m3, one fp32 scale per (seq, head))
 *   K nvfp4 : codes [16][d/2], then e4m3 block scales [16][d/16]
 *   V int8  : codes [d][16] (token-minor), then fp32 scale [16]
 *   V fp8   : codes [d][16]
 *   V nvfp4 : codes [d/2][16] (byte = elements 2i | 2i+1<<4 of one token), scales [d/16][16]
 *   K, V f32 / bf16 (unquantized): values [16][d] in the act dtype
 * Pools must be zero-filled once when allocated: slots of a page beyond the sequence length
 * are read (and masked) by the attention kernels and must hold finite bit patterns.
 * ---------------------------------------------------------------------------------- */
size_t tsb200_kv_record_bytes(int format, int head_dim);

typedef struct {
  int32_t format;        /* tsb200_kv_format                                            */
  int32_t hkv;           /* number of kv heads                                           */
  int32_t head_dim;      /* 64 or 128                                                    */
  int32_t reserved;
  int64_t num_pages;
  uint8_t* k_pool;       /* 16-byte aligned                                              */
  uint8_t* v_pool;
  const int32_t* block_table; /* [B, bt_stride]: page id of logical page i of sequence b */
  int64_t bt_stride;
  const int32_t* seq_lens;    /* [B] tokens currently in the cache                       */
  const float* k_scale;  /* fp8 only: [B, hkv]                                           */
  const float* v_scale;
} tsb200_kv_desc;

/* fp8 per-(sequence, head) scales from a prompt: scale = amax/448 (1.0 when amax == 0)
 * over k[b, :, h, :] (after the same RoPE the append applies when tables are given; token
 * j of sequence b is at position pos0[b] + j, pos0 NULL = 0) and over v[b, :, h, :].
 * k, v [B, T, hkv, d] act dtype.  Outputs fp32 [B, hkv]. */
int tsb200_kv_fp8_scales(const void* k, const void* v, int dtype, int64_t B, int64_t T,
                         int hkv, int head_dim, const int32_t* pos0,
                         const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                         float* k_scale, float* v_scale, void* stream);

/* Fused (RoPE on k +) quantize-and-append of T new tokens per sequence.
 * k, v [B, T, hkv, d]; token j of sequence b goes to position seq_lens[b] + j.
 * new_lens (int32 [B], may be NULL = T): only the first new_lens[b] tokens are appended.
 * rope_cos/rope_sin: fp32 tables [rope_rows, d/2] indexed by position, or NULL (k is
 * appended as given).  Rotation is the half-split form of blocks/rope.py:140-173 with
 * each product and sum rounded to the act dtype.  seq_lens is NOT modified.
 * Positions beyond the block table (>= bt_stride*16) are skipped.
 * k/v_token_stride: elements between consecutive tokens (0 = hkv*d, i.e. dense), so k and v
 * may be column slices of one fused [B*T, (H + 2 hkv) d] projection output. */
int tsb200_kv_append(const tsb200_kv_desc* kv, const void* k, const void* v, int dtype,
                     int64_t k_token_stride, int64_t v_token_stride,
                     int64_t B, int64_t T, const int32_t* new_lens,
                     const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                     void* stream);

/* tsb200_kv_append plus, in the same launch, the in-place RoPE of the query heads
 * q [B, T, q_heads, d] (token stride q_token_stride, 0 = dense) at the same positions
 * seq_lens[b] + j: the whole post-projection step of a decoder attention block
 * (blocks/mha.py:575-589) in one kernel.  q may be NULL (then identical to tsb200_kv_append);
 * a non-NULL q requires the rope tables. */
int tsb200_rope_append(const tsb200_kv_desc* kv, void* q, int q_heads, int64_t q_token_stride,
                       const void* k, const void* v, int dtype,
                       int64_t k_token_stride, int64_t v_token_stride,
                       int64_t B, int64_t T, const int32_t* new_lens,
                       const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                       void* stream);

/* Dequantizing gather: k_out, v_out [B, L, hkv, d] (act dtype) <- the first L positions of every
 * sequence, dequantized (fp8: times the sequence's scale); positions >= seq_lens[b] become zeros.
 * Serves attention reads over T > 1 query tokens (prefill with a library attention kernel): the
 * reference attends over the cache tensors themselves (blocks/mha.py:537-612; HF
 * past_key_values.update returns them), which for a quantized cache are its dequantized values.
 * L <= bt_stride * 16. */
int tsb200_kv_gather(const tsb200_kv_desc* kv, void* k_out, void* v_out, int dtype, int64_t B, int64_t L,
                     void* stream);

/* Prompt (prefill) attention.
 * Replaces blocks/mha.py:9-103 (attention()) for T > 1 query tokens per sequence - what the reference's model
 * classes hand to torch's scaled-dot-product attention while a prompt is processed - with causal masking: query i
 * of a sequence sits at position L - T + i and attends over positions 0 .. L - T + i of the cache.
 * Two steps.  tsb200_kv_gather_heads dequantizes the first L cached positions of every sequence into the layout
 * the attention kernel's copy engine wants: k_out [B, hkv, L, d] and vt_out [B, hkv, d, Lp] (V TRANSPOSED: the
 * tokens of one element are contiguous; Lp >= L is the row pitch, a multiple of 8; zeros beyond seq_lens[b] and in
 * [L, Lp)), both bf16.  tsb200_prefill_attn then runs the attention on tcgen05 (bf16 in, fp32 accumulation, bf16
 * out): q, out [B, T, H, d]; q_token_stride = elements between consecutive tokens of q (0 = H * d; a multiple of
 * 8), so q may be a column slice of a fused projection output; out is dense.  head_dim 64 or 128.  status: device
 * int32, set non-zero when a bounded wait ran out (may be NULL). */
int tsb200_kv_gather_heads(const tsb200_kv_desc* kv, void* k_out, void* vt_out, int64_t B, int64_t L, int64_t Lp,
                           void* stream);
int tsb200_prefill_attn(const void* q, int64_t q_token_stride, const void* k, const void* vt, void* out, int64_t B,
                        int64_t T, int64_t L, int64_t Lp, int H, int hkv, int head_dim, float sm_scale,
                        int32_t* status, void* stream);

/* Split-K paged decode attention: one query token per sequence.
 * Replaces blocks/mha.py:9-103 (attention(): GQA, softmax(q k^T / sqrt(d)) v) for the
 * decode step, reading the quantized pages directly.
 * q, out [B, H, d] act dtype; attends over seq_lens[b] tokens (0 -> zeros).
 * max_seq_len bounds seq_lens (sizes the split grid; lengths above it are clamped).
 * q_batch_stride: elements between consecutive sequences of q (0 = H*d); out is dense.
 * max_seq_len must not exceed bt_stride * 16 (the block table covers it) and num_pages must be positive,
 * else TSB200_ERR_ARG.
 * The first 16384 bytes of the workspace hold split counters and, in the last 4 of them (byte 16380), a
 * status word: zero-fill them ONCE before the first use; every completed call leaves the counters zero.
 * The status word becomes non-zero when a kernel gave up on a bounded wait for its own copies (the output
 * of that call is then not to be trusted); the caller reads and clears it.  One workspace must not serve
 * overlapping calls.
 * Arithmetic: scores and outputs accumulate in fp32.  The tensor-core kernels feed q and the softmax weights to the
 * MMA as f16 (int8 / NVFP4 pages) or as the sum of three e4m3 terms (FP8 pages, d = 128, <= 4 query heads per kv
 * head): about 11-12 significant bits either way, also when q and out are fp32.  Unquantized pages are attended in
 * fp32 throughout (tsb200_paged_decode_attn_simt, which accepts every format). */
size_t tsb200_paged_decode_attn_workspace_bytes(int64_t B, int H, int head_dim, int64_t max_seq_len);
int tsb200_paged_decode_attn(const tsb200_kv_desc* kv, const void* q, void* out, int dtype,
                             int64_t q_batch_stride, int64_t B, int H, float sm_scale, int64_t max_seq_len,
                             void* workspace, size_t workspace_bytes, void* stream);
/* Same contract; CUDA-core kernel (cross-check of the tensor-core kernel). */
int tsb200_paged_decode_attn_simt(const tsb200_kv_desc* kv, const void* q, void* out, int dtype,
                                  int64_t q_batch_stride, int64_t B, int H, float sm_scale, int64_t max_seq_len,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free decode attention.  (No counterpart in the reference: the reference lets
 * PyTorch allocate whatever it needs.)  Same contract and results as tsb200_paged_decode_attn,
 * but the split partials are kept in a fixed array inside the library, so the call needs no
 * workspace and performs no allocation of any kind.  It is meant for callers that cannot call
 * cudaMalloc on their serving path (fixed-budget plugins, runtimes whose allocator must not be
 * re-entered, code already inside a stream capture).
 *   - capacity: tsb200_paged_decode_attn_static_capacity() bytes (8 MiB); a problem whose split
 *     partials (16 KB + B * H * splits * (2 + head_dim) floats, splits as the library picks them for
 *     this B, hkv and max_seq_len - never more than tsb200_paged_decode_attn_workspace_bytes(...))
 *     exceed it is refused with TSB200_ERR_WORKSPACE.  Each GPU that loads the library holds the array
 *     until exit.
 *   - the first call on a device resolves the array's device address (cudaGetSymbolAddress with
 *     that device current); make that first call before any stream capture begins.
 *   - all calls on a device share the array: two calls that may overlap on the GPU (different
 *     streams) race.  The array keeps the previous call's contents.  Its first 16 KB (split counters and
 *     status word) have to be zero when the kernels start; since an overlapped or interrupted call could
 *     leave a counter stuck and the caller cannot reach the array, every call clears that head itself
 *     with a cudaMemsetAsync on `stream` ahead of its kernels (no allocation involved). */
size_t tsb200_paged_decode_attn_static_capacity(void);
int tsb200_paged_decode_attn_static(const tsb200_kv_desc* kv, const void* q, void* out, int dtype,
                                    int64_t q_batch_stride, int64_t B, int H, float sm_scale,
                                    int64_t max_seq_len, void* stream);

/* ------------------------------------------------------------------------------------
 * Small decoder ops
 * ---------------------------------------------------------------------------------- */
/* In-place half-split RoPE (blocks/rope.py:140-173) on x [B, T, heads, d]; position of
 * token (b, j) is pos0[b] + j (pos0 int32 [B], NULL = 0); token_stride = elements between
 * consecutive tokens (0 = heads*d). */
int tsb200_rope(void* x, int dtype, int64_t token_stride, int64_t B, int64_t T, int heads, int head_dim,
                const int32_t* pos0, const float* rope_cos, const float* rope_sin,
                int64_t rope_rows, void* stream);

/* residual += delta (delta may be NULL), then y = RMSNorm(residual) * w.
 * variant 0: Hugging Face Qwen2/Llama RMSNorm (fp32 x*rsqrt(mean(x^2)+eps), cast, *w);
 * variant 1: blocks/norm.py:8-23 (x /= max(1, max|x|), eps fixed 1e-5, in act dtype).
 * residual, delta, y [M, hidden]; w [hidden]. y may alias delta. */
int tsb200_add_rmsnorm(void* residual, const void* delta, const void* w, void* y, int dtype,
                       int64_t M, int64_t hidden, float eps, int variant, void* stream);

/* y = silu(gate) * up (blocks/mlp.py:181-183); gate, up, y [M, n] with row strides in
 * elements (so gate/up may be the two halves of one [M, 2n] buffer). */
int tsb200_swiglu(const void* gate, const void* up, void* y, int dtype, int64_t M, int64_t n,
                  int64_t gate_stride, int64_t up_stride, int64_t y_stride, void* stream);

/* ---------------------------------------------------------------- tensor-parallel epilogue -----
 * No reference counterpart (the reference is single-device).  One process per GPU; every rank's
 * buffers are mapped into the other ranks' address spaces by the host (CUDA IPC) and described by: */
typedef struct {
  int32_t world, rank;           /* 2..8 ranks; this process's index                                   */
  const void* partial[8];        /* partial[s]: rank s's [M, hidden] bf16 partial output ([rank] = local) */
  uint32_t* flags[8];            /* flags[s]: rank s's flag block, tsb200_peer_flag_bytes(), zero at start */
  uint32_t* epoch;               /* local: two uint32, zero at start                                     */
  int32_t* status;               /* local: non-zero after a peer failed to show up within the bounded wait */
} tsb200_peer_desc;
size_t tsb200_peer_flag_bytes(void);
/* cudaDeviceEnablePeerAccess from the current device to peer_device (idempotent). */
int tsb200_enable_peer_access(int peer_device);
/* IPC handle (64 bytes) of the cudaMalloc allocation that contains ptr, and ptr's byte offset in it. */
int tsb200_ipc_export(const void* ptr, void* handle64_out, uint64_t* offset_out);
/* Map / unmap an allocation that another process of this node exported with cudaIpcGetMemHandle
 * (handle64 = the 64 handle bytes) into the CURRENT device's address space; *base_out is the
 * address of the exported allocation's base. */
int tsb200_ipc_open(const void* handle64, void** base_out);
int tsb200_ipc_close(void* base);
/* residual += sum over ranks of partial_s (ranks in index order, fp32, rounded to bf16), then
 * y = RMSNorm(residual) * w (Hugging Face variant): the all-reduce that follows a row-parallel
 * LinearCompressed (o_proj, down_proj) fused with tsb200_add_rmsnorm, over NVLink peer loads.
 * bf16, hidden % 8 == 0, hidden <= 8192, M <= 1024.  Every rank must make the same sequence of calls
 * on the group, and must alternate between two partial buffers on consecutive calls (a buffer may be
 * rewritten only after the following call has started on every rank). */
int tsb200_peer_allreduce_add_rmsnorm(const tsb200_peer_desc* pd, void* residual, const void* w, void* y,
                                      int dtype, int64_t M, int64_t hidden, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TSB200_H */
