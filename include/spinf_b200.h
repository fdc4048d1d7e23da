/* spinf_b200: C ABI of the B200 (sm_100a) packed-prefill scoring kernels.
 *
 * The reference (spinf-serve) has no FFI of its own: its seams for this path are Python callables (attention interface, quantized
 * linear modules, the recurrent-layer functions, the scorer's lm-head read). Each entry point below is what a binding for one of
 * those seams calls; the comment above it names the reference symbol (file:line inside the spinf-serve tree) whose arithmetic it
 * replaces. Conventions:
 *   - plain pointers and sizes only; every pointer is DEVICE memory unless the name ends in _host;
 *   - `stream` is a cudaStream_t passed as void*; calls enqueue work and return without synchronising;
 *   - no entry point allocates device memory except spinf_init (one 256-byte status word per device); scratch is passed in by
 *     the caller and sized by the matching *_workspace_bytes query;
 *   - return value: 0 = enqueued; negative = rejected on the host before any launch (SPINF_ERR_*);
 *   - kernels never spin without bound: a wait that gives up writes a positive code to the per-device status word, which
 *     spinf_last_status() returns (and clears). Outputs of a call that reported a status are undefined.
 */
#ifndef SPINF_B200_H
#define SPINF_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPINF_ERR_BAD_ARGUMENT (-1) /* null pointer, size or alignment the kernel does not support */
#define SPINF_ERR_CUDA (-2)         /* a CUDA runtime call failed (no device, launch error) */
#define SPINF_ERR_TENSORMAP (-3)    /* the TMA descriptor could not be encoded (unaligned base or pitch) */
#define SPINF_ERR_TOO_LARGE (-4)    /* a size exceeds a documented maximum */

/* device status codes returned by spinf_last_status */
#define SPINF_ST_TIMEOUT_FULL 1
#define SPINF_ST_TIMEOUT_EMPTY 2
#define SPINF_ST_TIMEOUT_TMEM 3
#define SPINF_ST_TIMEOUT_OTHER 4
#define SPINF_ST_BAD_INDEX 5

#define SPINF_BLOCK 128 /* stream block size: packed streams are multiples of it (packer.py:22) */

/* Library version (major*10000 + minor*100 + patch). */
int spinf_version(void);

/* Prepares the current device: allocates its status word and raises the kernels' dynamic shared-memory limits. Call once per
 * device before any other entry point (and before any stream capture). */
int spinf_init(void);

/* Synchronises `stream`, returns the device status word (0 = every kernel since the last call completed its waits) and clears it. */
int spinf_last_status(void* stream);

/* Self-test of the error path every kernel of the library shares: launches one CTA that waits, for at most limit_ns (<= 1 s), on a
 * barrier nothing completes. The wait gives up, the kernel returns normally, and the next spinf_last_status reports
 * SPINF_ST_TIMEOUT_OTHER; the context stays usable. Nothing faults and nothing hangs. */
int spinf_selftest_bounded_wait(int64_t limit_ns, void* stream);

/* ------------------------------------------------------------------------------------------------------------ fp8 row-wise linear
 * Replaces quant_act_row (spinf_serve/quant/linears.py:29-33): per row m of x [M,K] bf16,
 *   xs[m] = max(|x[m,:]|, 1e-12) / 448 (fp32);  x8[m,k] = e4m3_rne(clamp(float(x[m,k]) / xs[m], -448, 448)).
 * K must be a multiple of 8 and at most 32768. */
int spinf_fp8_rowwise_quant(const void* x_bf16, int64_t M, int64_t K, void* x8, float* xs, void* stream);

/* Replaces Fp8RowLinear.forward's torch._scaled_mm call (spinf_serve/quant/linears.py:93-96):
 *   y[m,n] = bf16( (sum_k x8[m,k] * w8[n,k])_fp32 * xs[m] * ws[n] )
 * x8 [M,K] e4m3 row-major; w8 [N,K] e4m3 row-major (the storage of the reference's `w8t` buffer, which is the [K,N] column-major
 * view of it); xs [M], ws [N] fp32; y [M,N] bf16 row-major. K and N multiples of 16. A row of y does not depend on M. */
int spinf_fp8_rowwise_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M, int64_t N,
                           int64_t K, void* stream);

/* The same linear for a decoding step's few rows (M <= 128; the linears of the extraction decoder's steps,
 * spinf_serve/engine/decode.py:160-203, which the reference runs through the same torch._scaled_mm): the K dimension is cut into
 * slices, a function of N and K only, so that every SM streams weights; fp32 partial sums go to `workspace` (16-byte aligned, at
 * least spinf_fp8_rowwise_gemm_small_workspace_bytes), and a second launch adds them in slice order and applies the scales.
 * Differs from spinf_fp8_rowwise_gemm in the order of the fp32 sum only; ws 16-byte aligned. M > 128, or a shape whose column
 * tiles already cover the SMs (workspace bytes 0), runs spinf_fp8_rowwise_gemm. */
int64_t spinf_fp8_rowwise_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K);
int spinf_fp8_rowwise_gemm_small(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M, int64_t N,
                                 int64_t K, void* workspace, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------------------ fp8 per-tensor linears
 * The reference's Fp8Linear (dynamic) and Fp8StaticLinear (calibrated static activation scale, "fp8s"), both with one weight scale
 * per tensor (spinf_serve/quant/linears.py:66-119).
 *
 * spinf_abs_max: *out = max |x| over n bf16 elements (n a multiple of 8): the reduction of quant_act (linears.py:22-26). */
int spinf_abs_max(const void* x_bf16, int64_t n, float* out, void* stream);

/* x8[i] = e4m3_rne(clamp(float(x[i]) / s, -448, 448)) over n elements (a multiple of 8) with one scale read from device memory:
 *   from_amax = 0: s = *scale            (Fp8StaticLinear.forward, linears.py:113, scale = the module's `xs` buffer)
 *   from_amax = 1: s = max(*scale, 1e-12) / 448, *scale holding the tensor's max |x|      (quant_act, linears.py:22-26)
 * scale_out (may be NULL) receives s. peak (may be NULL): *peak = max(*peak, max|x| / (s * 448)), the clipping monitor of
 * Fp8StaticLinear (linears.py:111-112). */
int spinf_fp8_tensor_quant(const void* x_bf16, int64_t n, const float* scale, int32_t from_amax, void* x8, float* scale_out,
                           float* peak, void* stream);

/* Replaces the per-tensor torch._scaled_mm of Fp8Linear / Fp8StaticLinear (linears.py:77,114):
 *   y[m,n] = bf16( (sum_k x8[m,k] * w8[n,k])_fp32 * *xs * *ws ),   xs, ws: one fp32 each, in device memory.
 * Layouts and size rules as spinf_fp8_rowwise_gemm; the same kernel, so a row of y does not depend on M. */
int spinf_fp8_tensor_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M, int64_t N,
                          int64_t K, void* stream);

/* ------------------------------------------------------------------------------------------------------------ int8 linear (w8a8)
 * The reference's Int8Linear with int8 activations (spinf_serve/quant/linears.py:40-64, act8 = True).
 *
 * Replaces quant_act_int8 (linears.py:34-38): per row m of x [M,K] bf16,
 *   xs[m] = max(|x[m,:]|, 1e-12) / 127 (fp32);  x8[m,k] = int8(clamp(round_half_even(float(x[m,k]) / xs[m]), -127, 127)).
 * K must be a multiple of 8 and at most 32768. */
int spinf_int8_rowwise_quant(const void* x_bf16, int64_t M, int64_t K, void* x8, float* xs, void* stream);

/* Replaces torch._int_mm and the scaling after it (linears.py:61):
 *   y[m,n] = bf16( float(sum_k x8[m,k] * w8[n,k])_int32 * xs[m] * ws[n] )
 * x8 [M,K] int8 row-major; w8 [N,K] int8 row-major (the storage of the reference's `w8t` buffer); xs [M], ws [N] fp32; y [M,N]
 * bf16. K and N multiples of 16. Integer accumulation is exact, so a row of y depends on nothing but its own operands; unlike
 * torch._int_mm there is no lower limit on M (the reference pads to 17 rows, linears.py:59-60). */
int spinf_int8_rowwise_gemm(const void* x8, const float* xs, const void* w8, const float* ws, void* y_bf16, int64_t M, int64_t N,
                            int64_t K, void* stream);

/* The gate|up projection of a gated MLP with the activation fused into the GEMM epilogue (the reference runs
 * act(gate_proj(x)) * up_proj(x) as two Fp8RowLinear calls and an inductor-fused pointwise kernel: transformers' Gemma4TextMLP,
 * called through spinf_serve/models/gemma4.py:407-415; Qwen's MLP spinf_serve/models/qwen35/qwen.py:706-716):
 *   gate = bf16((x8 . wg)_fp32 * xs * ws_g), up likewise;  y[m,f] = bf16(bf16(act(gate[m,f])) * up[m,f]);  row_amax[m] = max_f |y[m,f]|
 * w8_tiled [2F, K] e4m3 / ws_tiled [2F] hold the gate and up channels in TILED order: for each group of 128 features, four
 * blocks of (32 gate rows, then the 32 up rows of the same features). y [M, F] bf16; row_amax [M] fp32 (cleared by the call).
 * F a multiple of 128, K a multiple of 16; act 0 = gelu (tanh form), 1 = silu. Same values as spinf_fp8_rowwise_gemm followed by
 * spinf_glu_quant. */
int spinf_fp8_rowwise_gemm_glu(const void* x8, const float* xs, const void* w8_tiled, const float* ws_tiled, void* y, float* row_amax,
                               int64_t M, int64_t F, int64_t K, int32_t act, void* stream);

/* The fused q|k|v projection of an attention layer with the per-head RMS norms and the rotary embedding applied in the GEMM
 * epilogue (the reference runs q_proj / k_proj / v_proj as Fp8RowLinear calls, then q_norm / k_norm / v_norm and
 * apply_rotary_pos_emb as inductor-fused pointwise kernels: transformers' Gemma4TextAttention, called through
 * spinf_serve/models/gemma4.py:383-405). w8 [(H + 2 Hkv) D, K] e4m3 holds the q heads, then the k heads, then the v heads; ws the
 * per-channel scales; wq / wk [D] bf16 the head-norm weights (plus1: scale by 1 + w); cos_t / sin_t [M, D/2] bf16 the rotary table
 * of the rows' positions (full rotary: the rotated width is D); norm_v: v heads get the weightless RMS norm. y [M, (H + 2 Hkv) D]
 * bf16. D is 128 or 256, (H + 2 Hkv) D a multiple of 256; y, wq, wk, cos_t, sin_t 32-byte aligned. Same values as
 * spinf_fp8_rowwise_gemm followed by spinf_qkv_norm_rope. */
int spinf_fp8_rowwise_gemm_qkv(const void* x8, const float* xs, const void* w8, const float* ws, void* y, int64_t M, int32_t H,
                               int32_t Hkv, int32_t D, int64_t K, const void* wq, const void* wk, const void* cos_t,
                               const void* sin_t, float eps, int32_t plus1, int32_t norm_v, void* stream);

/* Row-wise fp8 quantisation (arithmetic of spinf_fp8_rowwise_quant) of y [M, K] bf16 when the row maxima are already known:
 * xs[m] = max(row_amax[m], 1e-12) / 448, x8 = e4m3(clamp(y / xs)). One pass over y. */
int spinf_fp8_quant_from_amax(const void* y, const float* row_amax, int64_t M, int64_t K, void* x8, float* xs, void* stream);

/* Plain bf16 linear y = bf16(x @ w^T) with fp32 accumulation: x [M,K], w [N,K], y [M,N], all bf16 row-major; K, N multiples of 8.
 * Replaces the torch.nn.functional.linear / `x @ w.t()` calls on un-quantised weights (spinf_serve/models/qwen35/qwen.py:456-458
 * "extra" rows, and bf16-scheme linears). */
int spinf_bf16_gemm(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, void* stream);
/* The same with a row pitch for y (in elements, a multiple of 8): writes an [M, N] block inside a wider output, as the reference's
 * Int4Linear appends its un-quantised "extra" output channels to the int4 ones (spinf_serve/models/qwen35/qwen.py:421-426). */
int spinf_bf16_gemm_ld(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t y_pitch, void* stream);

/* spinf_bf16_gemm_ld for a decoding step's few rows (M <= 128) and few output channels (the un-quantised b | a rows beside an
 * Int4Linear, spinf_serve/models/qwen35/qwen.py:421-426,456-457, at a decoding step's rows): K in slices on separate CTAs, fp32
 * partial sums in `workspace` (16-byte aligned, at least spinf_bf16_gemm_small_workspace_bytes), added in slice order by a second
 * launch. Differs from spinf_bf16_gemm_ld in the order of the fp32 sum only; y 8-byte aligned, y_pitch a multiple of 4. A shape
 * that needs no slices (workspace bytes 0) runs spinf_bf16_gemm_ld. */
int64_t spinf_bf16_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K);
int spinf_bf16_gemm_small(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t y_pitch, void* workspace,
                          int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------------------ int4 weight-only linear
 * Replaces Int4Linear.forward in bf16 mode (spinf_serve/models/qwen35/qwen.py:455-458) with its per-call dequantisation dq_bf16
 * (qwen.py:326-330):  y[m,n] = bf16( sum_k x[m,k] * w[n,k] ),  w[n,k] = bf16( (nibble(n,k) - 8) * float(scales[n, k / group]) ).
 * x [M,K] bf16; qw uint8 [N, K/2] as spinf_w4_repack leaves it (below); scales fp16
 * [N, K/group]; y bf16 with row pitch y_pitch elements. The bf16 weight matrix is never materialised: nibbles are expanded inside
 * the kernel on their way to the tensor core. K a multiple of 64 and of group, group a multiple of 8 (128 in the benchmark
 * configuration, 32 in the reference's checkpoints), N a multiple of 8. A row of y does not depend on M. */
int spinf_w4_gemm(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                  int64_t y_pitch, void* stream);

/* spinf_w4_gemm for a decoding step's few rows (M <= 256): the same kernel with the K dimension cut into slices when the column
 * tiles alone do not occupy the GPU (out / down projections of 5 120 channels: 20 tiles for 74 CTA pairs); the slices' fp32 sums
 * go through `workspace` and are added in slice order before the one rounding to bf16, so a result may differ from spinf_w4_gemm's
 * in the last bf16 bit. Shapes that need no slices run spinf_w4_gemm itself. */
int64_t spinf_w4_gemm_small_workspace_bytes(int64_t M, int64_t N, int64_t K);
int spinf_w4_gemm_small(const void* x, const void* qw, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                        int64_t y_pitch, void* workspace, int64_t workspace_bytes, void* stream);

/* Load-time re-ordering of the packed int4 weights for spinf_w4_gemm. q_in: uint8 [N, K/2] in the reference's engine layout (byte b
 * of a row = k 2b in the low nibble, k 2b+1 in the high nibble: the `q` buffer of Int4Linear, qwen.py:383-389). q_out (may be
 * q_in): per 32-bit word of 8 consecutive k, the even k in nibbles 0..3 and the odd k in nibbles 4..7, so that the kernel takes a
 * pair (k, k+1) out of a word with one shift and one mask. Both 4-byte aligned, K a multiple of 8. */
int spinf_w4_repack(const void* q_in, void* q_out, int64_t N, int64_t K, void* stream);

/* Replaces the W4A16 linear of the extraction decoder's steps (spinf_serve/quant/w4gemm.py:17-66, `linear`): a few rows (M <= 128)
 * against int4 weights read as the engine stores them, streamed once. x [M, K] bf16 (rounded to fp16 as the reference does);
 * q uint8 [N, K/2] in the ENGINE layout (byte b = k 2b in the low nibble, k 2b + 1 in the high one; value nibble - 8; not
 * re-ordered by spinf_w4_repack); scales fp16 [N, K / group]. y[m, n] = bf16( sum over split-K partial sums, in split order, of
 * fp32 sums of fp16 products x[m, k] * fp16((nibble - 8) * scale) ); y bf16 with row pitch y_pitch. K a multiple of 256, group a
 * multiple of 32 that divides 256. The split count follows the reference (about 512 programs of 64 output channels). */
int64_t spinf_w4_small_workspace_bytes(int64_t M, int64_t N, int64_t K);
int spinf_w4_small(const void* x, const void* q, const void* scales, int32_t group, void* y, int64_t M, int64_t N, int64_t K,
                   int64_t y_pitch, void* workspace, int64_t workspace_bytes, void* stream);

/* The gate|up projection of a gated MLP with its activation in the GEMM epilogue: replaces Int4Linear.forward on the fused gate_up
 * weight followed by act(gate) * up (spinf_serve/models/qwen35/qwen.py:455-458 and the MLP around it, :700-712):
 *   y[m,c] = bf16( bf16(act(g)) * u ),  g = bf16(sum_k x[m,k] w[2c,k]),  u = bf16(sum_k x[m,k] w[2c+1,k]),   c < N2 / 2,
 * act = 0: GELU (tanh form), 1: SiLU. qw / scales hold the N2 = 2F rows INTERLEAVED (row 2c = gate channel c, row 2c+1 = up channel
 * c), each row as spinf_w4_repack leaves it. y [M, N2/2] bf16 with row pitch y_pitch. Other rules as spinf_w4_gemm; N2 a multiple
 * of 16. The [M, N2] intermediate is never written. */
int spinf_w4_gemm_glu(const void* x, const void* qw, const void* scales, int32_t group, int32_t act, void* y, int64_t M, int64_t N2,
                      int64_t K, int64_t y_pitch, void* stream);

/* ------------------------------------------------------------------------------------------------------------ option log-probs
 * Replaces Scorer._logprobs followed by the `[:, ci]` gather (spinf_serve/scorer.py:340-355 and :254): for read rows h [R,hidden]
 * bf16 and the lm-head matrix W [vocab,hidden] bf16,
 *   logits = h @ W^T (fp32 accumulate, fp32 out); if softcap > 0: logits = softcap * tanh(logits / softcap);
 *   out[r,c] = logits[r, cols[c]] - logsumexp_v(logits[r, v])            (fp32 [R, n_cols])
 * The [R,vocab] matrix is never written: the GEMM's epilogue keeps a running (max, sum-exp) per row and vocabulary tile and
 * captures the option columns. `cols` are the sorted (ascending) distinct option token ids (Scorer._cols, scorer.py:420-430), on
 * the device; an id outside [0, vocab) is skipped and its output column left unwritten. `workspace` needs spinf_option_logprobs_workspace_bytes(R, vocab, n_cols) bytes.
 * hidden a multiple of 8. A row's result does not depend on R (no padding to lm_rows is needed, scorer.py:327-333). */
int64_t spinf_option_logprobs_workspace_bytes(int64_t R, int64_t vocab, int64_t n_cols);
int spinf_option_logprobs(const void* h, const void* W, int64_t R, int64_t hidden, int64_t vocab, const int32_t* cols,
                          int64_t n_cols, float softcap, float* out, void* workspace,
                          int64_t workspace_bytes, void* stream);

/* Allocation-free variant of spinf_option_logprobs (it has no counterpart in the reference: the reference's lm-head read always
 * allocates its [rows, vocab] temporaries through torch). For callers that cannot allocate device memory at call time: a
 * serving process whose own allocator already owns all of HBM, a host-language binding with no device allocator, or a code path
 * where cudaMalloc's device-wide synchronisation is not acceptable. Same arithmetic and same result as spinf_option_logprobs;
 * the per-tile partial maxima / sums and the column table live in a fixed array inside the library image (8 MiB + 8 KiB,
 * resident on every GPU that loads the library until the process exits) instead of a caller workspace.
 *   - limit: 256 + 8 * ceil(vocab / 256) * (ceil(R / 128) * 128) + 4 * (ceil(vocab / 256) + 1) bytes must fit in that array
 *     (e.g. R <= 1024 rows at vocab 262144, R <= 2048 at vocab 131072); larger calls return SPINF_ERR_TOO_LARGE and launch nothing;
 *   - the call itself performs no cudaMalloc / cudaFree and calls no allocating routine; spinf_init is not required (the first
 *     call on a device also sets the kernel's shared-memory attribute, once);
 *   - the first call on a device resolves the array's device address (cudaGetSymbolAddress): make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array: the array keeps the previous call's contents, none of which is read before being
 *     rewritten, so back-to-back calls on one stream are safe; two calls that overlap on the GPU (different streams) race;
 *   - status: optional device pointer to one int32 the caller owns and has zeroed; a bounded wait that gives up stores its code
 *     there (SPINF_ST_*). NULL = not reported (the code lands in a slot of the array that nothing reads back). */
int spinf_option_logprobs_static(const void* h, const void* W, int64_t R, int64_t hidden, int64_t vocab, const int32_t* cols,
                                 int64_t n_cols, float softcap, float* out, int32_t* status, void* stream);

/* ------------------------------------------------------------------------------------------------------------ tree-mask attention
 * Host function. Replaces packer.block_tables (spinf_serve/packer.py:426-491): from the per-token arrays of
 * a packed stream (art, end, pos: int32 [n], n a multiple of 128) builds, for each 128-row query block, the ascending list of
 * 128-column key blocks it must visit and a flag byte per entry: bit 0 = "full" in the reference's classification (every pair
 * attends; never set on the sliding table), bit 1 = the kernel may skip the mask evaluation (every pair attends, window included).
 *   counts_host [nb], blocks_host [nb*nb] (row i holds counts[i] entries), flags_host [nb*nb] (uint8).
 * window <= 0: full-attention table; window > 0: sliding table (no "full" flags, blocks wholly outside the window skipped).
 * Returns the total number of visited blocks, or a negative error. */
int64_t spinf_tile_desc_build_host(const int32_t* art_host, const int32_t* end_host, const int32_t* pos_host, int64_t n,
                                   int32_t window, int32_t* counts_host, int32_t* blocks_host, uint8_t* flags_host);

/* The same for streams with images (block_tables' `grp` argument, packer.py:455-467,479,485): grp_host [n] int32 = the image a
 * placeholder token belongs to, -1 elsewhere (NULL: a text-only stream). A sliding-table tile is kept when its two blocks share an
 * image even if the window would skip it, and a query block also visits the LATER key blocks of its images (partial tiles, listed
 * after the diagonal, ascending). */
int64_t spinf_tile_desc_build_host_img(const int32_t* art_host, const int32_t* end_host, const int32_t* pos_host, const int32_t* grp_host,
                                       int64_t n, int32_t window, int32_t* counts_host, int32_t* blocks_host, uint8_t* flags_host);

/* The mask rule of the packed stream (spinf_serve/scorer.py:173-177, the mask_mod the reference hands to create_block_mask) evaluated
 * once per stream and mask type instead of once per layer and head: for entry e of the packed tile lists, key half hf (0 / 1) and
 * row r of the entry's query block, bit c of bits[(e * 2 + hf) * 128 + r] = visible(128 qb + r, 128 j + 64 hf + c) as defined below.
 * art / end / pos, tile_offsets / tile_blocks on the device; bits: 2 * 128 * (number of entries) uint64 on the device. */
int spinf_tile_mask_bits(const int32_t* art, const int32_t* end, const int32_t* pos, int64_t n, int32_t window,
                         const int32_t* tile_offsets, const int32_t* tile_blocks, uint64_t* bits, void* stream);

/* The mask rules of streams with images (spinf_serve/scorer.py:178-198, the `full_img` / `sliding_img` mask_mods): visible(t, k) of
 * spinf_tile_mask_bits, or grp[t] >= 0 && grp[k] == grp[t] (an image's placeholder tokens see each other both ways), with
 * grp_in_window != 0 only when also pos[t] - pos[k] < window (the sliding layers of models whose global layers stay causal: those
 * pass grp = NULL for their full-attention table). grp [n] int32 on the device, NULL = spinf_tile_mask_bits. The tile lists must
 * come from spinf_tile_desc_build_host_img with the same grp. */
int spinf_tile_mask_bits_img(const int32_t* art, const int32_t* end, const int32_t* pos, const int32_t* grp, int64_t n, int32_t window,
                             int32_t grp_in_window, const int32_t* tile_offsets, const int32_t* tile_blocks, uint64_t* bits,
                             void* stream);

/* Replaces the "tree_flex" attention interface (spinf_serve/models/gemma4.py:99-121, mask rule spinf_serve/scorer.py:173-177) and
 * qwen.tree_attention (spinf_serve/models/qwen35/qwen.py:605-623):
 *   out[t,h,:] = sum_k softmax_k(scale * q[t,h,:].k[k,g,:] | visible(t,k)) v[k,g,:],   g = h / (H/Hkv)
 *   visible(t,k) = (k <= t && art[t] >= 0 && art[k] == art[t] && t < end[k] && (window <= 0 || pos[t]-pos[k] < window)) || t == k
 * q [n,H,D], k,v [n,Hkv,D], out [n,H,D] bf16, token-major with row pitches given in ELEMENTS (so q/k/v may be slices of one fused
 * projection output); D in {128, 256}; n a multiple of 128. tile_offsets [nb+1] (prefix sums of counts), tile_blocks, tile_flags:
 * the packed lists from spinf_tile_desc_build_host, on the device; tile_bits: the visibility words of spinf_tile_mask_bits for the
 * same lists and window (entries flagged "no mask" are not read). Scores are fp32, P is rounded to bf16 before P.V, the running
 * maximum is updated once per 128 keys in ascending key order: a row's result depends only on its own job's tokens. scale > 0;
 * out 32-byte aligned with a row pitch that is a multiple of 16 elements. row_amax: NULL, or [n] fp32 zeroed by the caller: receives
 * max |out[t,:,:]| per token (the row maximum the fp8 quantiser of the output projection's input needs: spinf_fp8_quant_from_amax). */
int spinf_tree_attn_fwd(const void* q, const void* k, const void* v, void* out, int64_t n, int32_t H, int32_t Hkv, int32_t D,
                        int64_t q_pitch, int64_t kv_pitch, int64_t out_pitch, const int32_t* art, const int32_t* end,
                        const int32_t* pos, int32_t window, float scale, const int32_t* tile_offsets, const int32_t* tile_blocks,
                        const uint8_t* tile_flags, const uint64_t* tile_bits, float* row_amax, void* stream);

/* ------------------------------------------------------------------------------------------------------------ layer glue
 * The reference runs these steps as inductor-fused pieces of the decoder layer (the layer code itself is the transformers
 * Gemma 4 text model the reference instantiates at spinf_serve/models/gemma4.py:134-143 and calls at :407-415; Qwen's own layer
 * at spinf_serve/models/qwen35/qwen.py:502-510,699-734). Each entry point fuses a chain of them so an activation row crosses HBM
 * once; rounding points are the modules' (every module output bf16, norms in fp32).
 *
 * spinf_fused_norm: per output row r (input row rows[r] when `rows` is given, else r) of y [*, hidden] bf16:
 *   a = y;  if w1: a = bf16(a * (mean(a^2) + eps)^-1/2 * w1);  if residual: a = bf16(a + residual[r]);  out_h[r] = a (optional);
 *   if w2: b = bf16(rmsnorm(a) * w2) -> out_norm[r] (optional) and/or its per-row fp8 quantisation out_x8[r], out_xs[r]
 *   (the arithmetic of spinf_fp8_rowwise_quant). plus1: weights enter as (1 + w). hidden a multiple of 8, at most 8192. */
int spinf_fused_norm(const void* y, const int64_t* rows, const void* w1, const void* residual, const void* w2, int64_t n_out,
                     int64_t hidden, float eps, int32_t plus1, void* out_h, void* out_norm, void* out_x8, float* out_xs,
                     void* stream);

/* In place on the fused q|k|v projection output qkv [n, pitch] bf16 (H query heads, then Hkv key heads, then Hkv value heads, D
 * each): per head RMSNorm (q with wq [D], k with wk [D], v without weight when norm_v) rounded to bf16, then the rotary embedding
 * of q and k over the first rot_dim dimensions, bf16(bf16(x cos) + bf16(rotate_half(x) sin)), with cos_t / sin_t [n, rot_dim/2]
 * bf16 from spinf_rope_table. D in {128, 256}; rot_dim a multiple of D/16. */
int spinf_qkv_norm_rope(void* qkv, int64_t pitch, int64_t n, int32_t H, int32_t Hkv, int32_t D, const void* wq, const void* wk,
                        const void* cos_t, const void* sin_t, int32_t rot_dim, float eps, int32_t plus1, int32_t norm_v,
                        void* stream);

/* The Qwen attention layer's layout (spinf_serve/models/qwen35/qwen.py:683-697): the fused projection row is
 * [H x (q (D) | gate (D))] | k (Hkv D) | v (Hkv D). Query heads are normed (RMSNorm with (1 + w) when plus1) and rotated over the
 * first rot_dim dimensions like spinf_qkv_norm_rope and written DENSE to q_out [n, H, D]; key heads are normed and rotated in
 * place; value heads and gates are left untouched. */
int spinf_qkv_norm_rope_gated(void* y, int64_t pitch, int64_t n, int32_t H, int32_t Hkv, int32_t D, const void* wq, const void* wk,
                              const void* cos_t, const void* sin_t, int32_t rot_dim, float eps, int32_t plus1, void* q_out,
                              void* stream);

/* In place o[t,h,:] = bf16(o[t,h,:] * bf16(sigmoid(gate[t,h,:]))), gate read from the same interleaved projection rows y (column
 * h * 2 D + D): the output gate of the Qwen attention layer (qwen.py:696). o [n, H, D] bf16 dense. */
int spinf_attn_gate(void* o, const void* y, int64_t pitch, int64_t n, int32_t H, int32_t D, void* stream);

/* cos_t / sin_t [n, rot_dim/2] bf16 = bf16(cos / sin (float(pos[t]) * inv_freq[f])), inv_freq [rot_dim/2] fp32 on the device. */
int spinf_rope_table(const int32_t* pos, int64_t n, int32_t rot_dim, const float* inv_freq, void* cos_t, void* sin_t, void* stream);

/* gu [n, 2F] bf16 = gate | up (one fused projection): y = bf16(bf16(act(gate)) * up), act 0 = gelu (tanh form), 1 = silu; then
 * its per-row fp8 quantisation (out_x8 [n,F], out_xs [n]) and/or y itself in bf16 (out_y [n,F]). F a multiple of 8. */
int spinf_glu_quant(const void* gu, int64_t n, int64_t F, int32_t act, void* out_x8, float* out_xs, void* out_y, void* stream);

/* out[t,:] = bf16(emb[ids[t],:] * scale): the scaled word embedding (ids int64; an id outside [0, vocab) reads row 0). */
int spinf_embed_scale(const int64_t* ids, const void* emb, int64_t n, int64_t hidden, int64_t vocab, float scale, void* out,
                      void* stream);

/* ------------------------------------------------------------------------------------------------------------ Gated DeltaNet
 * Replaces gdn.recurrent and gdn.chunked (spinf_serve/models/qwen35/gdn.py:197-235 and :109-133; the per-token arithmetic is
 * gdn.py:176-186) with their calling contract: the n_seg segments of one plan call (cu [n_seg+1] int64, token t of the call =
 * row idx[t] of the stream tensors, or row t when idx is NULL), per segment and value head a state S [K, V] fp32 that starts
 * from h0[h0_idx[seg]] (zero when h0 is NULL or the index is negative) and is written to ht[ht_idx[seg]] where that index is >= 0:
 *     S *= exp(g);  v' = (v - S^T k) * beta;  S += k (x) v';  o = S^T (q * scale)
 * q, k [rows, Hk, K] bf16 (l2-normalised by the caller), v [rows, Hv, V] bf16, g fp32 / beta bf16 [rows, Hv], each with its row
 * pitch in elements (g and beta share g_pitch); o [rows, Hv, V] bf16 contiguous, written at the same rows; h0 / ht
 * [*, Hv, K, V] fp32. K = V = 128; Hv and g_pitch even, q / k / v 16-byte aligned with pitches that are multiples of 8 elements.
 * Token-serial: any segment length is accepted; segments longer than 64 tokens are meant for
 * spinf_gdn_chunked below. */
int spinf_gdn_recurrent(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o, int64_t n_rows,
                        int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V, float scale,
                        const int64_t* cu, int64_t n_seg, const int64_t* idx, const float* h0, const int64_t* h0_idx, float* ht,
                        const int64_t* ht_idx, void* stream);

/* The same recurrence for long segments in the chunked (WY) form the reference switches to above 64 tokens (gdn.chunked,
 * spinf_serve/models/qwen35/gdn.py:109-133, which runs flash-linear-attention 0.5.2's chunk pipeline: chunk_local_cumsum,
 * chunk_gated_delta_rule_fwd_intra, the state kernel of gdn.py:21-106, chunk_fwd_o). Same arguments as spinf_gdn_recurrent, plus the
 * chunk table of the call (64-token chunks, segments in order: chunk_seg [n_chunks] = segment, chunk_t0 [n_chunks] = first token of
 * the chunk within its segment; int32 on the device), call_tokens = cu[n_seg], and a workspace of
 * spinf_gdn_chunked_workspace_bytes(call_tokens, Hv) bytes (16-byte aligned) for W, U and the running log-decay. Operands of every
 * product are rounded to bf16 and accumulated in fp32, the state stays fp32, as in the reference's pipeline; results differ from
 * the token-serial form by those roundings. */
int64_t spinf_gdn_chunked_workspace_bytes(int64_t call_tokens, int32_t Hv);
int spinf_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o, int64_t n_rows,
                      int64_t q_pitch, int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V, float scale,
                      const int64_t* cu, int64_t n_seg, const int64_t* idx, const float* h0, const int64_t* h0_idx, float* ht,
                      const int64_t* ht_idx, const int32_t* chunk_seg, const int32_t* chunk_t0, int64_t n_chunks,
                      int64_t call_tokens, void* workspace, int64_t workspace_bytes, void* stream);

/* A whole trie plan in the chunked form: replaces the reference's per-level driver gdn_indexed and the kernels it calls
 * (spinf_serve/models/qwen35/qwen.py:550-590; gdn.py:109-133 and :197-235) for one recurrent layer. Every segment of the plan,
 * long or short, runs in chunks of at most 64 tokens with the rounding points of spinf_gdn_chunked; a segment's values depend
 * only on its own tokens and its parent's final state. The host describes the plan once per stream (gdn_plan.fused_schedule):
 *   row_of [plan_tokens] int64   stream (or compact) row of plan token p; plan order = the segments one after the other
 *   chunk_p0 / chunk_len [n_chunks] int32   every chunk of every segment: first plan token, length (1..64)
 * spinf_gdn_tree_prep (ONE launch for the layer: nothing in it depends on a state) fills the workspace of
 * spinf_gdn_tree_workspace_bytes(plan_tokens, Hv) bytes (256-byte aligned): W, U [plan_tokens, Hv, 128] bf16,
 * P [plan_tokens, Hv, 64] bf16, G [plan_tokens, Hv] fp32.
 * spinf_gdn_tree_scan runs one level of the trie (levels in order, after prep, on the same stream): the level's segments are
 * grouped by parent; group i reads the parent's final state h_in[grp_parent[i]] (negative: the zero state) once and walks its units
 * grp_ubeg[i] .. grp_ubeg[i+1]. A unit is 12 int32 words: number of pieces (1..4), flags (1 = the chunk updates the state, 2 =
 * the unit must see the parent's state), the row of h_out the state is stored to after the update (-1: none), a pad word, and
 * per piece (first plan token, length). Pieces are children that only read the state (one chunk, no state to keep), laid out at
 * 16-row-aligned offsets of one 64-row tile; a child with several chunks, or whose state a deeper level reads, is one unit per
 * chunk with flag 1 (its first with flags 1 | 2). h_in / h_out [slots, Hv, 128, 128] fp32. Outputs o [rows, Hv, 128] bf16
 * contiguous at the tokens' rows. q / k / v / g / beta as for spinf_gdn_recurrent. */
int64_t spinf_gdn_tree_workspace_bytes(int64_t plan_tokens, int32_t Hv);
int spinf_gdn_tree_prep(const void* q, const void* k, const void* v, const float* g, const void* beta, int64_t n_rows, int64_t q_pitch,
                        int64_t v_pitch, int64_t g_pitch, int32_t Hk, int32_t Hv, int32_t K, int32_t V, const int64_t* row_of,
                        int64_t plan_tokens, const int32_t* chunk_p0, const int32_t* chunk_len, int64_t n_chunks, void* workspace,
                        int64_t workspace_bytes, void* stream);
int spinf_gdn_tree_scan(const void* q, const void* k, void* o, int64_t n_rows, int64_t q_pitch, int32_t Hk, int32_t Hv, int32_t K,
                        int32_t V, float scale, const int64_t* row_of, int64_t plan_tokens, const int32_t* grp_parent,
                        const int32_t* grp_ubeg, const int32_t* units, int64_t n_groups, const float* h_in, float* h_out,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* spinf_gdn_tree_scan on the 5th-generation tensor cores: the same units, arithmetic and rounding points, with tcgen05.mma on
 * 128-byte-swizzled operand tiles in shared memory and the state (whole 128 x 128, no column slices) in tensor memory for the
 * CTA's lifetime. Takes the workspace spinf_gdn_tree_prep filled, and unit_rows [units, 4, 64] int32, the units' rows spelled
 * out by the host: per row its plan token (-1: no token), its stream row (< 2^31), the plan token of its piece's last token, its
 * piece's first row. Every wait inside the kernel is bounded; one that gives up is reported through spinf_last_status. */
int spinf_gdn_tree_scan_tc(const void* q, const void* k, void* o, int64_t n_rows, int64_t q_pitch, int32_t Hk, int32_t Hv, int32_t K,
                           int32_t V, float scale, int64_t plan_tokens, const int32_t* grp_parent, const int32_t* grp_ubeg,
                           const int32_t* units, const int32_t* unit_rows, int64_t n_groups, const float* h_in, float* h_out,
                           void* workspace, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------- extraction decoder's attention
 * Replaces `_x_attention` (spinf_serve/decode.py:71-104), the attention of a batched decoding step: G groups, Q slots each (one new
 * token per slot), H query heads over h key/value heads of D. Token-major tensors, all bf16:
 *   q   rows (g * Q + slot) of q_pitch elements, head j at offset j * D          out  the same shape, row pitch out_pitch
 *   kp, vp [G, Lp, h, D]  the groups' prefixes, pos_p [G, Lp] int32 positions (-1: padding, never attended)
 *   kt, vt [G, Tt, h, D]  the templates, pos_t their positions, own_t [G, Tt] the owning prompt (-1: padding): slot s attends to
 *                         the tokens of prompt s / beam only
 *   gk, gv [G, Q, S, h, D] the tokens generated by each slot's own beam: tokens 0 .. *step are attended (step: int32 on the device,
 *                         so that a captured launch can be replayed at the next step). k_new, v_new (both or neither): the step's
 *                         own K / V rows (row g * Q + slot of kv_pitch elements, head j at j * D), written into gk / gv at token
 *                         *step before they are attended: GroupKV.update (decode.py:60-65) inside the same launch
 *   qpos [G, Q] int32 the queries' positions; window > 0 also hides keys with qpos - pos >= window (sliding layers)
 * Rounding points as the reference: scores rounded to bf16 before scaling, soft cap (0: none) and mask; softmax in fp32 over the
 * three ranges together; probabilities rounded to bf16; each range's value product rounded to bf16, the three added in fp32. */
int64_t spinf_x_attention_workspace_bytes(int64_t G, int64_t Q, int64_t H, int64_t D, int64_t Lp, int64_t Tt, int64_t S);
int spinf_x_attention(const void* q, int64_t q_pitch, const void* kp, const void* vp, const int32_t* pos_p, int64_t Lp,
                      const void* kt, const void* vt, const int32_t* pos_t, const int32_t* own_t, int64_t Tt, void* gk, void* gv,
                      int64_t S, const void* k_new, const void* v_new, int64_t kv_pitch, const int32_t* qpos, const int32_t* step,
                      int64_t G, int64_t Q, int64_t H, int64_t h,
                      int64_t D, int32_t beam, int32_t window, float scale, float softcap, void* out, int64_t out_pitch,
                      void* workspace, int64_t workspace_bytes, void* stream);

/* Replaces the steps of GatedDeltaNet.forward before the recurrence (spinf_serve/models/qwen35/qwen.py:651-668), fused: for each of
 * the T tokens, from the in-projection rows y [n_rows, y_pitch] bf16 = [q | k | v | z | b | a]: the 4-tap path convolution over
 * conv [T, 4] int64 (a tap index >= n_rows or < 0 is the zero row) with conv_w [2 Hk K + Hv V, 4] bf16 in fp32, SiLU, rounding
 * to bf16; q and k then l2-normalised per head (x * rsqrt(sum x^2 + 1e-6)); beta = bf16(sigmoid(b));
 * g = -exp(A_log) * softplus(a + dt_bias) in fp32. Outputs q, k [T, Hk, K], v [T, Hv, V] bf16, g [T, Hv] fp32, beta [T, Hv] bf16. */
int spinf_gdn_prologue(const void* y, int64_t y_pitch, int64_t n_rows, int64_t T, const int64_t* conv, const void* conv_w,
                       const float* A_log, const float* dt_bias, int32_t Hk, int32_t Hv, int32_t K, int32_t V, void* q, void* k,
                       void* v, float* g, void* beta, void* stream);

/* Replaces the gated RMS norm after the recurrence (spinf_serve/models/qwen35/qwen.py:670-673): per token and value head
 * of = o * rsqrt(mean(o^2) + eps); out = bf16(float(bf16(norm_w * bf16(of))) * silu(z)). o [T, Hv, V] bf16 contiguous, z rows of
 * pitch z_pitch (a slice of the in-projection output), norm_w [V] bf16, out [T, Hv V] bf16. */
int spinf_gdn_epilogue(const void* o, const void* z, int64_t z_pitch, const void* norm_w, float eps, int64_t T, int32_t Hv, int32_t V,
                       void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPINF_B200_H */
