/* libmfx — C ABI of the B200 (sm_100a) quantized DiT denoising-step kernels.
 *
 * The reference (filipstrand/mflux) has no native boundary of its own: its hot path is a chain of
 * Python-level MLX calls. Each entry point below replaces one of those calls; the comment above it
 * names the reference call site (path inside the reference project : line).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer owned by the caller, unless a comment says "host";
 *  - every call enqueues work on `stream` (a cudaStream_t passed as void*) and returns at once;
 *  - the return value is 0 (MFX_OK) or a negative mfx_status; nothing throws across this boundary;
 *  - the library allocates no device memory; shapes and alignments are validated on the host
 *    before anything is launched;
 *  - bounded device-side waits report through mfx_poll_device_status() instead of hanging;
 *  - threads: every entry point may be called from several host threads, and for several devices of one process
 *    (the few per-device records the library keeps - kernel attributes, SM count, the address of the static
 *    scratch - sit under mutexes); calls act on the device that is current in the calling thread. What the library
 *    does not order is the caller's own memory: two calls that write the same workspace or output, a prepared blob
 *    that is being rebuilt while another stream reads it, or the one static scratch must be ordered by the caller.
 */
#ifndef MFX_H_
#define MFX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MFX_VERSION 100

typedef enum mfx_status {
  MFX_OK = 0,
  MFX_ERR_SHAPE = -1,            /* a size is zero/negative or violates a divisibility rule */
  MFX_ERR_ALIGN = -2,            /* a pointer or stride is not 16-byte aligned where required */
  MFX_ERR_UNSUPPORTED_BITS = -3, /* bits not in {3, 4, 5, 6, 8} or group size != 64 */
  MFX_ERR_DTYPE = -4,            /* dtype code not accepted by this entry point */
  MFX_ERR_ARCH = -5,             /* current device is not compute capability 10.x */
  MFX_ERR_CUDA = -6,             /* a CUDA runtime/driver call failed (see mfx_last_cuda_error) */
  MFX_ERR_NULL = -7,             /* a required pointer is NULL */
  MFX_ERR_DEVICE_TIMEOUT = -8,   /* a bounded device-side wait gave up (mfx_poll_device_status) */
  MFX_ERR_TOO_LARGE = -9         /* a size exceeds a documented fixed limit */
} mfx_status;

typedef enum mfx_dtype { MFX_F32 = 0, MFX_BF16 = 1, MFX_F16 = 2 } mfx_dtype;

/* Quantizer flavour. MFX_QMODE_MLX: the algorithm MLX ships (scale oriented towards the extreme of
 * larger magnitude and snapped so that 0.0 is exactly representable). MFX_QMODE_DOC: the formula of
 * MLX's documentation, scale=(max-min)/(2^bits-1), bias=min. */
typedef enum mfx_qmode { MFX_QMODE_MLX = 0, MFX_QMODE_DOC = 1 } mfx_qmode;

/* Epilogues fused into the quantized matmul (v = acc + bias). */
typedef enum mfx_epilogue {
  MFX_EPI_NONE = 0,          /* y = v */
  MFX_EPI_GELU_ERF = 1,      /* y = gelu(v), erf form        (mlx.nn.gelu) */
  MFX_EPI_GELU_TANH = 2,     /* y = gelu(v), tanh form       (mlx.nn.gelu_approx) */
  MFX_EPI_GATE_RESIDUAL = 3, /* y = residual + gate[sample] * v */
  MFX_EPI_SILU = 4,          /* y = v * sigmoid(v) */
  MFX_EPI_PEER_SCATTER = 6,  /* tensor parallel: the bf16 product (no bias) of a linear split along K is not written
                                to y but scattered, row by row, into partial-sum slots in the memory of the rank
                                that owns each row (mfx_qlinear_args.scatter); mfx_tp_fuse sums the slots */
  MFX_EPI_SWIGLU = 5         /* y[:, j] = silu(v[:, 2j]) * v[:, 2j+1]; y is N/2 wide, N % 16 == 0. The caller
                                interleaves the rows of the gate and up projections (w1 row j -> row 2j, w3 row j
                                -> row 2j+1), which turns silu(w1 x) * (w3 x) of the reference's FeedForward
                                (src/mflux/models/z_image/model/z_image_transformer/feed_forward.py:13-14) into
                                one matmul */
} mfx_epilogue;

int mfx_version(void);
const char* mfx_status_str(int status);
/* Text of the last CUDA error this library saw on the calling thread ("" if none). */
const char* mfx_last_cuda_error(void);
/* Reads and clears the device status word written by bounded waits. *status_out = 0 when clean,
 * else a positive code naming the wait that gave up. Synchronises `stream`. */
int mfx_poll_device_status(int* status_out, void* stream);

/* Replaces mx.quantize(w, group_size=64, bits) as reached through mlx.nn.quantize from
 * src/mflux/models/common/weights/loading/weight_applier.py:93-103.
 * w [N, K] row-major (w_dtype) -> wq uint32 [N, K*bits/32], scales/biases [N, K/64] in w_dtype.
 * bits is 3, 4, 5, 6 or 8 (the widths of src/mflux/cli/defaults/defaults.py:63). Code j of a row occupies bits
 * [j*bits, (j+1)*bits) of the row's little-end-first bit stream: 8 or 4 codes per uint32 at 4 / 8 bits, codes
 * straddling byte and word boundaries at 3, 5 and 6 bits (8 codes in 3 or 5 bytes, 4 codes in 3 bytes). */
int mfx_quantize_affine(const void* w, int w_dtype, int64_t N, int64_t K, int bits, int group_size, int qmode,
                        uint32_t* wq, void* scales, void* biases, void* stream);

/* Replaces mx.dequantize (used when a quantized layer is read back as dense weights, e.g. LoRA baking,
 * src/mflux/models/common/lora/mapping/lora_saver.py). out [N, K] in out_dtype = q*scale + bias. */
int mfx_dequantize_affine(const uint32_t* wq, const void* scales, const void* biases, int sb_dtype, int64_t N,
                          int64_t K, int bits, int group_size, void* out, int out_dtype, void* stream);

/* Kernel-side ("prepared") form of one quantized weight. The matmul kernel streams weights and
 * per-group scale/bias pairs with TMA and dequantizes with the fewest integer instructions when
 *  (a) the codes of each uint32 are interleaved so that one mask yields two neighbouring values
 *      (4 bits: nibble order e0,e2,e4,e6,e1,e3,e5,e7; 8 bits: byte order e0,e2,e1,e3), and
 *  (b) scales and biases are transposed and paired: sb[g*N + n] = bf16(scales[n,g]) | bf16(biases[n,g]) << 16.
 * Codes of 3 bits are widened to 4 and codes of 5 or 6 bits to 8 on the way, so the matmul kernels unpack two
 * widths only (kb = 4 or 8); the matmul is bound by the tensor cores at every width, so the wider stream costs no time.
 * Scales and biases are carried as bf16 whatever sb_dtype is: f16 / f32 scales lose mantissa bits here (each
 * dequantized weight moves by at most 2^-9 of scale and bias), which MLX's quantized_matmul does not do.
 * The blob is [interleaved codes, N*K*kb/8 bytes, padded to 256][sb, (K/64)*N*4 bytes]. It has no
 * counterpart in the reference (MLX consumes its own [N, K*bits/32] / [N, K/64] arrays directly); a
 * caller that keeps weights resident prepares once per weight and passes `prepared` afterwards. */
size_t mfx_qlinear_prepared_bytes(int64_t N, int64_t K, int bits, int group_size); /* 0 on bad arguments */
int mfx_qlinear_prepare(const uint32_t* wq, const void* scales, const void* biases, int sb_dtype, int64_t N,
                        int64_t K, int bits, int group_size, void* prepared, size_t prepared_bytes, void* stream);

/* Replaces mlx.nn.QuantizedLinear.__call__ = mx.quantized_matmul(x, w, scales, biases, transpose=True,
 * group_size=64, bits) + bias, i.e. every nn.Linear of the transformer blocks, e.g.
 * src/mflux/models/flux/model/flux_transformer/joint_attention.py:14-21, feed_forward.py:8-9,
 * single_transformer_block.py:14-15.
 * y[M, N] = x[M, K] . dequant(wq)^T + bias.  x bf16 with row stride ldx (elements, multiple of 8);
 * y bf16 or f32 with row stride ldy; bias nullable. K % 64 == 0, N % 8 == 0.
 * workspace: caller-owned scratch of mfx_qlinear_prepared_bytes(N, K, bits, 64) bytes, 256-byte aligned;
 * the call first prepares the weight into it (see above), then runs the matmul, both on `stream`. */
int mfx_qlinear(const void* x, int64_t M, int64_t K, int64_t ldx, const uint32_t* wq, const void* scales,
                const void* biases, int sb_dtype, int64_t N, int bits, int group_size, const void* bias,
                int bias_dtype, void* y, int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes,
                void* stream);

/* Allocation-free form of mfx_qlinear. It has no counterpart in the reference. It exists for callers that
 * cannot hand the library a workspace because they cannot allocate device memory at the point of the call:
 * a serving process whose allocator reserved all of HBM at start-up, a plugin host that forbids
 * allocations inside its execution callbacks, a latency-critical loop that cannot afford the implicit
 * device synchronisation of cudaMalloc/cudaFree. The scratch that mfx_qlinear takes as `workspace` is
 * instead a fixed array of MFX_STATIC_SCRATCH_BYTES inside the library image; each GPU that loads the
 * library holds it until the process exits. The call allocates nothing.
 *  - Limit: mfx_qlinear_prepared_bytes(N, K, bits, 64) <= MFX_STATIC_SCRATCH_BYTES (e.g. a 12288 x 3072
 *    weight at 4 bits needs 21.2 MB); larger weights return MFX_ERR_TOO_LARGE and nothing is launched.
 *  - The first call on a device looks up the array's device address (once per device, with that device
 *    current); make that first call before any stream capture begins.
 *  - All calls share the one array and each call overwrites the part it uses, so nothing has to be cleared
 *    between calls; but two calls that overlap on the GPU (different streams, or another thread) race on
 *    it. Serialise them, or use mfx_qlinear with separate workspaces. */
#define MFX_STATIC_SCRATCH_BYTES (32 * 1024 * 1024)
int mfx_qlinear_static_scratch(const void* x, int64_t M, int64_t K, int64_t ldx, const uint32_t* wq,
                               const void* scales, const void* biases, int sb_dtype, int64_t N, int bits,
                               int group_size, const void* bias, int bias_dtype, void* y, int y_dtype, int64_t ldy,
                               void* stream);

/* Strided, batched form with fused epilogues. The activations are `batch` samples of `rows` rows:
 * element (b, r, k) at x + b*x_batch_stride + r*x_row_stride + k; y and residual likewise; gate is
 * [batch, N] with gate_batch_stride. This lets the joint text+image blocks read/write slices of one
 * sequence buffer without concatenation copies (joint_attention.py:57-60,75-79) and fuses the gated
 * residual of joint_transformer_block.py:84-90 / single_transformer_block.py:45,56-57.
 * Weights: either `prepared` (from mfx_qlinear_prepare; then wq/scales/biases may be NULL) or
 * wq + scales + biases + a workspace as in mfx_qlinear. */
/* Tensor-parallel exchange (no counterpart in the single-device reference; it serves the column- / row-split
 * QuantizedLinear layers of the Qwen-Image blocks, qwen_transformer_block.py:27-76, when one image is spread over
 * several GPUs). Every rank owns rows_per_rank consecutive rows of each sample's joint sequence. All pointers in
 * dst / flags are addresses valid on THIS device: the peers' buffers mapped into this process (peer access or
 * symmetric memory), entry r belonging to rank r. Peers are written with ordinary stores only. */
#define MFX_TP_MAX_WORLD 8
typedef struct mfx_tp_scatter {
  int world, rank;
  int64_t rows_per_rank; /* R: rows of a sample's joint sequence owned by one rank */
  int64_t row_offset;    /* joint-sequence row of this call's first activation row */
  int64_t D;             /* width of a partial row (= N of the linear) */
  void* dst[MFX_TP_MAX_WORLD];  /* on rank r: bf16 slots [world, batch, R, D]; this rank writes slot [rank] */
  int* flags[MFX_TP_MAX_WORLD]; /* on rank r: the counter this rank bumps by one when all its rows are out */
  int* done_counter;     /* local int, zero between calls (counts finished thread blocks) */
} mfx_tp_scatter;

typedef struct mfx_qlinear_args {
  const void* x;            /* bf16 */
  int64_t x_row_stride, x_batch_stride;
  int64_t rows, batch, K, N;
  const uint32_t* wq;
  const void* scales;
  const void* biases;
  int sb_dtype, bits, group_size;
  const void* prepared;      /* nullable */
  void* workspace;           /* nullable when prepared is given */
  size_t workspace_bytes;
  const void* bias;         /* nullable, [N] */
  int bias_dtype;
  int epilogue;             /* mfx_epilogue */
  const void* gate;         /* [batch, N], required for MFX_EPI_GATE_RESIDUAL */
  int gate_dtype;
  int64_t gate_batch_stride;
  const void* residual;     /* same dtype as y, required for MFX_EPI_GATE_RESIDUAL */
  int64_t res_row_stride, res_batch_stride;
  void* y;
  int y_dtype;              /* MFX_BF16 or MFX_F32 */
  int64_t y_row_stride, y_batch_stride;
  /* Optional low-rank term, added to the product before bias and epilogue (lora_r == 0: none). Replaces
   * `scale * (x @ lora_A) @ lora_B` of LoRALinear.__call__ (src/mflux/models/common/lora/layer/
   * linear_lora_layer.py:50-53) and the sum over adapters of FusedLoRALinear.__call__
   * (fused_linear_lora_layer.py:13-20): the caller passes t = x @ [A_1 | A_2 | ...] and
   * lora_b[n, :] = [scale_1 * B_1[:, n] | scale_2 * B_2[:, n] | ...]; the kernel runs them as extra K columns
   * of the same tensor-core accumulation. Both are bf16 with rows of lora_ld values (a multiple of 64, at most
   * 1024); columns at and after lora_r must be zero. */
  const void* lora_t;       /* [batch, rows, lora_ld] */
  int64_t lora_t_row_stride, lora_t_batch_stride;
  const void* lora_b;       /* [N, lora_ld], dense */
  int64_t lora_ld;
  int64_t lora_r;
  const mfx_tp_scatter* scatter; /* host pointer; required for MFX_EPI_PEER_SCATTER (then y may be NULL) */
} mfx_qlinear_args;
int mfx_qlinear_ex(const mfx_qlinear_args* args /* host */, void* stream);

/* The elementwise half of a tensor-parallel block on the rows this rank owns, fused with both collectives:
 *   wait until rs_flags[r] >= rs_target for every rank r (the partials of the preceding row-split linears),
 *   x += gate * (sum_r partials[r] + bias)          (qwen_transformer_block.py:56-57,64,69)
 *   n = LayerNorm(x, eps) * (1 + scale) + shift      (the next sub-layer's modulated pre-norm, :35-47)
 *   store n (bf16) at its joint row in push_dst[r] for every rank r, then add 1 to *ag_flags[r].
 * partials == NULL skips the wait and the residual update (first norm of the first block); scale == NULL for both
 * segments skips norm and push (after the last block). Segment 0 are joint rows < split (text stream), segment 1
 * the others (image stream): each has its own bias, gate, shift and scale. Rows at or beyond seq are padding. */
typedef struct mfx_tp_fuse_args {
  int world, rank;
  int64_t batch, rows_per_rank, seq_pad /* = world * rows_per_rank */, seq, split, D;
  float* x;             /* [batch, rows_per_rank, D] float32 residual rows of this rank, updated in place */
  const void* partials; /* local bf16 [world, batch, rows_per_rank, D], or NULL */
  const int* rs_flags;  /* local [world] */
  int rs_target;        /* waited-for value = rs_target + (epoch_base ? epoch_base[0] : 0) */
  const int* epoch_base; /* local int the caller advances between steps (so that a recorded CUDA graph of a step
                            can be replayed: the counters only grow), or NULL */
  const void* bias[2];  /* [D], nullable */
  int bias_dtype;
  const void* gate[2];  /* [batch, D] */
  const void* shift[2];
  const void* scale[2];
  int mod_dtype;        /* of gate, shift, scale */
  int64_t mod_batch_stride;
  float eps;
  void* push_dst[MFX_TP_MAX_WORLD]; /* on rank r: bf16 [batch, seq_pad, D] */
  int* ag_flags[MFX_TP_MAX_WORLD];  /* on rank r: the counter this rank bumps */
  int* done_counter;    /* local int, zero between calls */
  int push_local_only;  /* 1: store n into push_dst[rank] only and bump no counter: the caller moves the rows to the
                           peers itself (e.g. with the copy engines, beside the next matmul) and then calls
                           mfx_tp_signal */
} mfx_tp_fuse_args;
int mfx_tp_fuse(const mfx_tp_fuse_args* args /* host */, void* stream);
/* Adds 1 to *flags[r] for r < world with system-scope release semantics: the arrival signal of rows that were moved
 * to the peers by stream-ordered copies enqueued before this call on the same stream. `flags` is a host array. */
int mfx_tp_signal(int* const* flags /* host */, int world, void* stream);
/* Enqueues a wait until flags[r] >= target + (epoch_base ? *epoch_base : 0) for r < world (local counters that
 * peers bump). The wait is bounded: after about a second it gives up and mfx_poll_device_status reports it. */
int mfx_tp_wait(const int* flags, int world, int target, const int* epoch_base, void* stream);

/* Replaces nn.LayerNorm(affine=False, eps)(x) * (1 + scale) + shift
 * (src/mflux/models/flux/model/flux_transformer/ada_layer_norm_zero.py:20, ada_layer_norm_zero_single.py:17,
 * joint_transformer_block.py:86-87, ada_layer_norm_continuous.py:19) and, with rms=1, nn.RMSNorm(weight, eps)
 * optionally followed by the same modulation (z_image_transformer/transformer_block.py:29-34,
 * qwen_transformer_rms_norm.py:11-23). x is `batch` samples of `rows` rows of D values (f32 or bf16),
 * shift/scale are [batch, D] (nullable), weight is [D] (nullable); y is bf16. D % 8 == 0, D <= 4096. */
typedef struct mfx_norm_args {
  const void* x;
  int x_dtype;
  int64_t x_row_stride, x_batch_stride;
  int64_t rows, batch, D;
  const void* shift;
  const void* scale;
  int mod_dtype;
  int64_t mod_batch_stride;
  const void* weight;
  int weight_dtype;
  float eps;
  int rms; /* 0 = LayerNorm with biased variance, 1 = RMSNorm */
  void* y; /* bf16 */
  int64_t y_row_stride, y_batch_stride;
} mfx_norm_args;
int mfx_norm_modulate(const mfx_norm_args* args /* host */, void* stream);

/* Replaces AttentionUtils.process_qkv's per-head nn.RMSNorm(128) on Q and K plus AttentionUtils.apply_rope
 * (src/mflux/models/flux/model/flux_transformer/common/attention_utils.py:30-34,75-80), in place on the
 * fused activation buffer qkv [batch, seq, >= 3*heads*128] bf16 laid out q | k | v per token. Rows
 * s < split use the (qw_a, kw_a) norm weights (text stream: norm_added_q/k), the others (qw_b, kw_b).
 * cos_sin is f32 [seq, 64, 2] = (cos, sin) of each rotated (even, odd) pair (embed_nd.py:19-31). */
int mfx_qknorm_rope(void* qkv, int64_t row_stride, int64_t batch_stride, int64_t seq, int64_t batch, int heads,
                    int64_t split, const void* qw_a, const void* kw_a, const void* qw_b, const void* kw_b,
                    int w_dtype, const float* cos_sin, float eps, void* stream);

/* The same with fewer key heads than query heads and a choice of rotary layout: the buffer holds q (heads) |
 * k (kv_heads) | v (kv_heads) per token. Replaces Krea2QKNorm + Krea2RopeEmbedder.apply_rope on the projections of
 * Krea2Attention (src/mflux/models/krea2/model/krea2_transformer/attention.py:25-35, common.py:19-28,
 * rope_embedder.py:31-37: the same rotation of (even, odd) pairs, rope_mode 0; the caller passes the norm weights as
 * scale + 1, common.py:13-14), and norm_q / norm_k + apply_rotary_emb of ErnieAttention
 * (src/mflux/models/ernie_image/model/ernie_transformer/attention.py:42-46, rope_embedder.py:31-37), rope_mode 1:
 * x * cos + (-x[64:], x[:64]) * sin, where element j of either half reads angle j / 2 of cos_sin[s] (the embedder
 * stores every angle twice, rope_embedder.py:24-28). */
int mfx_qknorm_rope_gqa(void* qkv, int64_t row_stride, int64_t batch_stride, int64_t seq, int64_t batch, int heads,
                        int kv_heads, int rope_mode, int64_t split, const void* qw_a, const void* kw_a,
                        const void* qw_b, const void* kw_b, int w_dtype, const float* cos_sin, float eps,
                        void* stream);

/* y[b, r, :] *= act(gate[b, r, :]) on bf16 rows of D elements (D a multiple of 8, strides in elements). act 0 =
 * sigmoid: the output gate of Krea2Attention, `out * mx.sigmoid(gate)` in front of `wo`
 * (krea2_transformer/attention.py:41); act 1 = GELU (erf): `up_proj(x) * nn.gelu(gate_proj(x))` of ErnieFeedForward
 * (src/mflux/models/ernie_image/model/ernie_transformer/feed_forward.py:12-13). */
int mfx_act_mul(void* y, int64_t y_row_stride, int64_t y_batch_stride, const void* gate, int64_t g_row_stride,
                int64_t g_batch_stride, int64_t rows, int64_t batch, int64_t D, int act, void* stream);

/* Replaces mx.fast.scaled_dot_product_attention(q, k, v, scale) without mask
 * (attention_utils.py:48-52) for head dimension 128: softmax(Q K^T * scale) V per (sample, head).
 * q, k, v are bf16 views [batch, seq, heads, 128] given by their token and batch strides (elements), e.g.
 * the three sections of the fused qkv buffer; out is bf16 [batch, seq, heads*128] with its own strides,
 * which is the layout AttentionUtils.compute_attention returns after its transpose + reshape. */
int mfx_fmha(const void* q, const void* k, const void* v, int64_t qkv_row_stride, int64_t qkv_batch_stride,
             int64_t seq, int64_t batch, int heads, float scale, void* out, int64_t out_row_stride,
             int64_t out_batch_stride, void* stream);

/* mfx_fmha with an additive bias per key: softmax(Q K^T * scale + key_bias[sample, key]) V, the bias shared by
 * all heads and queries of a sample. Replaces scaled_dot_product_attention(..., mask=additive) where the mask is
 * the [B, 1, 1, S] key-padding mask built by AttentionUtils.convert_key_padding_mask_to_additive_mask
 * (attention_utils.py:55-72) and QwenAttention._convert_mask_for_qwen
 * (src/mflux/models/qwen/model/qwen_transformer/qwen_attention.py:117-135): 0 on real keys, -1e9 on padded text
 * keys. key_bias is f32 [batch, seq] with bias_batch_stride elements between samples (16-byte aligned, stride a
 * multiple of 4). Any finite values are accepted; a row whose keys all carry -1e9 yields the mean of V. */
int mfx_fmha_bias(const void* q, const void* k, const void* v, int64_t qkv_row_stride, int64_t qkv_batch_stride,
                  int64_t seq, int64_t batch, int heads, float scale, const float* key_bias,
                  int64_t bias_batch_stride, void* out, int64_t out_row_stride, int64_t out_batch_stride,
                  void* stream);

/* The same attention with its general shape: a key / value sequence of its own length and fewer key / value heads
 * than query heads. Replaces scaled_dot_product_attention as called
 *  - with keys and values that carry cached reference tokens behind the current ones, so seq_kv > seq_q
 *    (Flux2KVCache.append_reference, src/mflux/models/flux2/model/flux2_transformer/flux2_kv_cache.py:51-61, used by
 *    flux2_transformer/attention.py:69-72 and parallel_self_attention.py:46-49);
 *  - after mx.repeat(k / v, heads // kvheads, axis=1), i.e. grouped-query attention
 *    (src/mflux/models/krea2/model/krea2_transformer/attention.py:33-38): query head h reads key / value head
 *    h / (heads / kv_heads), nothing is repeated in memory.
 * q is bf16 [batch, seq_q, heads, 128], k and v bf16 [batch, seq_kv, kv_heads, 128] (row / batch strides in
 * elements, k and v share theirs), key_bias optional f32 [batch, seq_kv] as for mfx_fmha_bias, out bf16
 * [batch, seq_q, heads * 128]. heads must be a multiple of kv_heads. */
typedef struct mfx_fmha_args {
  const void* q;
  const void* k;
  const void* v;
  int64_t q_row_stride, q_batch_stride;
  int64_t kv_row_stride, kv_batch_stride;
  int64_t seq_q, seq_kv, batch;
  int heads, kv_heads;
  float scale;
  const float* key_bias;       /* NULL: no bias */
  int64_t bias_batch_stride;
  void* out;
  int64_t out_row_stride, out_batch_stride;
} mfx_fmha_args;
int mfx_fmha_ex(const mfx_fmha_args* args /* host */, void* stream);

/* out = act(a + b + c) elementwise (b, c nullable; act 0 = identity, 1 = SiLU, 2 = tanh): the conditioning-vector
 * arithmetic of time_text_embed.py:25-31, the nn.silu in front of every AdaLN linear and the mx.tanh on the
 * Z-Image gates (z_image_transformer/transformer_block.py:26-27). */
int mfx_vec_sum_act(const void* a, const void* b, const void* c, int in_dtype, int act, void* out, int out_dtype,
                    int64_t n, void* stream);

/* out = residual + gate[sample] * (y + bias): the gated residual of joint_transformer_block.py:84-90 /
 * qwen_transformer_block.py:56-57,64,69 as a stand-alone kernel, for tensor-parallel row-split linears whose
 * partial sums are all-reduced before the gate can be applied (no counterpart in the single-device reference).
 * y is [batch, rows, D] bf16 or f32 (dense), gate [batch, D], bias [D] nullable; residual and out are f32
 * [batch, rows, D] views that share their row and batch strides in elements (they may be the same view, or a row
 * range of the residual stream when the linear is evaluated in chunks). */
int mfx_gate_residual(const void* y, int y_dtype, const void* bias, int bias_dtype, const void* gate, int gate_dtype,
                      int64_t gate_batch_stride, const float* residual, float* out, int64_t res_row_stride,
                      int64_t res_batch_stride, int64_t batch, int64_t rows, int64_t D, void* stream);

/* residual += gate[sample] * RMSNorm(y) * weight, in place on the float32 residual stream: the post-norms
 * attention_norm2 / ffn_norm2 of src/mflux/models/z_image/model/z_image_transformer/transformer_block.py:31,35
 * (gate = tanh of the modulation, applied by the caller) and context_block.py:18,21 (gate == NULL).
 * y is [batch, rows, D] bf16 or f32 given by its strides (elements), gate [batch, D], weight [D], D % 8 == 0,
 * D <= 4096. */
int mfx_norm_gate_residual(const void* y, int y_dtype, int64_t y_row_stride, int64_t y_batch_stride, int64_t rows,
                           int64_t batch, int64_t D, const void* weight, int weight_dtype, float eps,
                           const void* gate, int gate_dtype, int64_t gate_batch_stride, float* residual,
                           int64_t res_row_stride, int64_t res_batch_stride, void* stream);

/* mfx_norm_gate_residual followed, in the same pass, by the pre-norm of the next sub-layer on the updated stream:
 * next_out = RMSNorm(residual) * next_weight * (1 + next_scale[sample]) as bf16, i.e. ffn_norm1 and scale_mlp after
 * the attention post-norm (transformer_block.py:34 after :31) or the following block's attention_norm1 and
 * scale_msa after the FFN post-norm (:29-30 after :35). next_out == NULL leaves only the first stage. */
typedef struct mfx_post_pre_norm_args {
  const void* y;
  int y_dtype;
  int64_t y_row_stride, y_batch_stride;
  int64_t rows, batch, D;
  const void* weight;
  int weight_dtype;
  float eps;
  const void* gate; /* [batch, D] or NULL */
  int gate_dtype;
  int64_t gate_batch_stride;
  float* residual;
  int64_t res_row_stride, res_batch_stride;
  void* next_out; /* bf16 [batch, rows, D] or NULL */
  int64_t next_row_stride, next_batch_stride;
  const void* next_weight;
  int next_weight_dtype;
  const void* next_scale; /* [batch, D] or NULL */
  int next_scale_dtype;
  int64_t next_scale_batch_stride;
  float next_eps;
} mfx_post_pre_norm_args;
int mfx_post_pre_norm(const mfx_post_pre_norm_args* args /* host */, void* stream);

/* Classifier-free-guidance combine of two noise predictions [rows, channels] into f32 `out`.
 * mode 0: noise + g*(noise - negative)  (src/mflux/models/z_image/variants/z_image.py:209);
 * mode 1: negative + g*(noise - negative), rescaled per row to the norm of `noise`
 *         (QwenImage.compute_guided_noise, src/mflux/models/qwen/variants/txt2img/qwen_image.py:165-174). */
int mfx_cfg_combine(const void* noise, const void* noise_negative, int dtype, float guidance, int mode, float* out,
                    int64_t rows, int64_t channels, void* stream);

/* Replaces LinearScheduler.step (src/mflux/models/common/schedulers/linear_scheduler.py:56-58):
 * out = latents + noise * dt, in the latents' dtype. */
int mfx_euler_step(const void* latents, int lat_dtype, const void* noise, int noise_dtype, float dt, void* out,
                   int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MFX_H_ */
