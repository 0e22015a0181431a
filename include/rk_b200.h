/*
 * rk_b200 - C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point
 *   - takes plain device pointers, sizes and a CUDA stream (a cudaStream_t passed as void*),
 *   - launches on that stream and returns without synchronising,
 *   - never allocates, frees or synchronises device memory (the caller owns every buffer,
 *     including the scratch "workspace"), so calls can be captured in a CUDA graph.  Two
 *     exceptions, both test aids: rk_read_status synchronises the stream and copies one word
 *     back; rk_probe_rcp_approx_448 allocates one word, runs on the default stream and synchronises;
 *     and the four rk_peer_* set-up calls, whose job is to allocate and map exchange memory,
 *   - returns RK_OK (0) or a negative RK_E* code; rk_last_error_string() describes the last
 *     failure on the calling thread.
 * There is no CPU fallback: unsupported shapes are errors.
 *
 * Each declaration names the reference interface it stands in for (path inside the reference
 * project : line).
 *
 * Data conventions
 *   bf16      : IEEE bfloat16, row-major, innermost stride 1
 *   int8 data : [rows, Kpad], Kpad = K rounded up to 128, zero padded
 *   int4 data : [rows, Kpad/2] bytes, two's-complement nibbles, low nibble = even k
 *   e4m3      : OCP FP8 E4M3 (no inf, max 448)
 *   SF buffer : block scale factors in 512-byte chunks of 128 rows x 4 factors; factor g of
 *               row r lives at ((r/128)*kt + g/4)*512 + (r%32)*16 + ((r%128)/32)*4 + g%4,
 *               kt = ceil(groups/4); size rk_sf_bytes(rows, groups)
 */
#ifndef RK_B200_H_
#define RK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RK_OK 0
#define RK_EINVAL (-1)      /* bad argument: null pointer, shape, alignment */
#define RK_EUNSUPPORTED (-2) /* shape or device this build has no kernel for */
#define RK_ECUDA (-3)       /* a CUDA runtime / driver call failed */
#define RK_EWORKSPACE (-4)  /* workspace missing or too small */
#define RK_EDEVICE (-5)     /* a kernel reported a bounded-wait expiry in the status word */

/* Activation pre-ops of the row quantizer (reference: MODE of `_prepare`, ampere_ada/integer.py:52-72). */
#define RK_ACT_PLAIN 0     /* v = x */
#define RK_ACT_LUT_MUL 1   /* v = bf16(LUT[bits(x)] * up) */
#define RK_ACT_LUT 2       /* v = LUT[bits(x)] */

/* GEMM families, for rk_workspace_bytes(). */
#define RK_OP_W8A8 0
#define RK_OP_W4A4 1
#define RK_OP_W4A16 2
#define RK_OP_FP8 3
#define RK_OP_MXFP8 4
#define RK_OP_NVFP4 5

/* Bytes at the start of every workspace reserved for the device status word. */
#define RK_WORKSPACE_HEADER 256

/* ---- library ---------------------------------------------------------------------------- */

/* Library ABI version (major*1000 + minor). */
int rk_version(void);
/* Description of the last error on this thread ("" when none). */
const char* rk_last_error_string(void);
/* 1 when the kernels can run on a device of this compute capability (10.0 only).
 * Reference: `supports_device`, blackwell/csrc/mxfp8_cutlass_linear.cu:275-277. */
int rk_supports_device(int cc_major, int cc_minor);
/* Size of the scratch buffer a GEMM call of this family and shape may use.  The buffer must be
 * zero-filled once after allocation; kernels leave it zero-filled.  One buffer per stream. */
size_t rk_workspace_bytes(int op, int64_t m, int64_t n, int64_t k);
/* Size of a swizzled scale-factor buffer for `rows` rows and `groups` factors per row.
 * Reference: `scale_storage_size`, blackwell/csrc/mxfp8_common.cuh:14-16. */
size_t rk_sf_bytes(int64_t rows, int64_t groups);
/* Reads (synchronously, after synchronising `stream`) and clears the device status word at the
 * start of `workspace`; workspace == NULL reads the status word of the scratch array built into the
 * library (rk_gemm_int4_noalloc) on the current device.  Returns RK_OK or RK_EDEVICE; *code
 * receives the raw device code. */
int rk_read_status(void* workspace, int* code, void* stream);
/* Test aid for the give-up path of the kernels' bounded waits (no reference counterpart).  While
 * `on` is non-zero, the tensor-core GEMM entry points rk_gemm_int / _fp8 / _mxfp8 / _nvfp4 launch
 * with every wait limited to `spin_limit` polls (64..2^21) and with a first pipeline stage that is
 * announced larger than what is copied, so its wait runs out: the kernel records a code in the
 * status word, drains and returns normally (nothing traps; the context stays usable), and
 * rk_read_status returns RK_EDEVICE.  Process-wide; switch it off again with on = 0. */
int rk_debug_wait_expiry(int on, int spin_limit);
/* Bit pattern of rcp.approx.ftz.f32(448.0f) on the current device (synchronous; test aid for the
 * MXFP8 block-scale formula, blackwell/csrc/mxfp8_common.cuh:25). */
int rk_probe_rcp_approx_448(uint32_t* bits);

/* ---- integer path ----------------------------------------------------------------------- */

/* Per-row symmetric absmax quantization of bf16 rows to int8 / packed int4.
 * Replaces `prepare_activation` + Triton `_prepare` (ampere_ada/integer.py:75-198).
 *   x [rows, k] with row stride x_stride (elements); up (RK_ACT_LUT_MUL only) likewise;
 *   lut: 65536 bf16 entries indexed by the bf16 bit pattern (modes 1, 2), else NULL;
 *   q: int8 [rows, kpad] (bits 8) or uint8 [rows, kpad/2] (bits 4); scales: f32 [rows].
 *   scale = max|v| * fl32(1/limit) (1.0 for a zero row), q = clamp(rint(v / scale)). */
int rk_quant_rows(const void* x, int64_t rows, int64_t k, int64_t x_stride, const void* up, int64_t up_stride,
                  const void* lut, int mode, int bits, void* q, float* scales, void* stream);

/* Per-output-channel weight quantization with true division (scale = max|w| / limit).
 * Replaces the torch ops of `IntegerLinear.from_linear` (ampere_ada/integer.py:247-263).
 *   w bf16 [n, k] contiguous; q int8 [npad, kpad] / uint8 [npad, kpad/2]; scales f32 [npad];
 *   npad = n rounded up to 8; padding rows get zero codes and scale 1.0. */
int rk_quant_weight_int(const void* w, int64_t n, int64_t k, int bits, void* q, float* scales, void* stream);

/* AdaLN modulation (optionally preceded by a gated residual add and a non-affine LayerNorm)
 * fused into the row quantizer.  Replaces `prepare_modulation`, `prepare_norm_modulation`,
 * `prepare_residual_norm_modulation` (ampere_ada/modulation.py:13-146, 149-236).
 *   x [rows, k]; scale, shift [rows/tokens, k] (row r uses row r / tokens);
 *   v = bf16(bf16(x' * bf16(1 + scale)) + shift), x' = x, LayerNorm(x) or LayerNorm(residual);
 *   y, gate (both or neither): residual = bf16(x + bf16(y * gate)) is written to residual_out;
 *   layer_norm != 0 applies LayerNorm with `eps` first. */
int rk_quant_rows_modulated(const void* x, const void* scale, const void* shift, int64_t rows, int64_t k,
                            int64_t tokens, int layer_norm, float eps, const void* y, const void* gate,
                            void* residual_out, int bits, void* q, float* scales, void* stream);

/* Gemma RMSNorm fused into the int8 / int4 row quantizer:
 *   s = x, or bf16(x + residual);  inv = rsqrt(mean(s^2) + eps);
 *   v = bf16( fl(fl(s * inv) * fl(1 + a)) (+ b) ),  every fl() an fp32 rounding;
 *   plain norm:    a = scale[k] (the learned weight), shift = NULL, tokens = 0;
 *   adaptive norm: a = scale[r / tokens, k], b = shift[r / tokens, k].
 * The norm is models/pi05/modeling_gemma.py:62-106; the reference has no fused integer version,
 * its precedent is `add_rms_norm_quantize_bf16` (blackwell/csrc/fp8_cutlass_linear.cu:145-269).
 *   sum_out (bf16 [rows, k], may be NULL) receives s; norm_out (may be NULL) receives v. */
int rk_rmsnorm_quant_rows(const void* x, const void* residual, const void* scale, const void* shift,
                          int64_t tokens, int64_t rows, int64_t k, float eps, int bits, void* sum_out,
                          void* norm_out, void* q, float* scales, void* stream);

/* The same with the gated residual of the adaptive layers in front (the reference's gated residual,
 * common/fused.py:47-58, is a kernel of its own, and its residual + norm + modulation + quantize
 * fusion exists for LayerNorm only: ampere_ada/modulation.py:149-265):
 *   s = bf16( x + bf16(branch * gate[r / tokens, k]) ), then as rk_rmsnorm_quant_rows.
 *   branch bf16 [rows, k]; gate bf16 [rows/tokens, k]; tokens >= 1; sum_out receives s. */
int rk_gated_rmsnorm_quant_rows(const void* x, const void* branch, const void* gate, const void* scale,
                                const void* shift, int64_t tokens, int64_t rows, int64_t k, float eps, int bits,
                                void* sum_out, void* norm_out, void* q, float* scales, void* stream);

/* The same Gemma RMSNorm (plain residual add, plain or adaptive weights) without a row quantizer:
 * writes the bf16 result to norm_out and, when scale_out is given, the per-tensor scale
 * max(amax(result) / divisor, 1e-12) of that result (non-finite values ignored) - the first half
 * of norm -> per-tensor-scaled FP8 / NVFP4 packing (divisor 448 or 6 * 448) in front of
 * rk_quant_tensor_fp8_with_scale or rk_pack_nvfp4.  The arithmetic is the model's norm
 * (models/pi05/modeling_gemma.py:62-106), not the two-rounding form of the reference's serving
 * producers (`add_rms_norm_fp4_quant_bf16`), so a stack keeps its numerics when it switches this on.
 *   scale_out == NULL: norm only (workspace unused); otherwise a workspace header is needed. */
int rk_rmsnorm_tensor_scale(const void* x, const void* residual, const void* scale, const void* shift, int64_t tokens,
                            int64_t rows, int64_t k, float eps, float divisor, void* sum_out, void* norm_out,
                            float* scale_out, void* workspace, size_t workspace_bytes, void* stream);

/* out[r, c] = bf16(table[x[r, c]] * up[r, c]) - the gated-activation arithmetic of rk_quant_rows'
 * RK_ACT_LUT_MUL mode (ampere_ada/integer.py:101-130: a 65536-entry bf16 table indexed by the bit
 * pattern) written as a bf16 matrix - and, when scale_out is given, max(amax(out) / divisor, 1e-12):
 * the activation in front of a down projection whose packer needs a per-tensor scale (NVFP4 with
 * global scales: divisor 6 * 448; FP8 per tensor: 448).
 *   x, up bf16 rows of k elements, row strides in elements (multiples of 8); out bf16 [rows, k]
 *   contiguous; k % 8 == 0; scale_out == NULL: product only (workspace unused). */
int rk_lut_mul_tensor_scale(const void* x, int64_t x_stride, const void* up, int64_t up_stride, const void* lut,
                            int64_t rows, int64_t k, float divisor, void* out, float* scale_out, void* workspace,
                            size_t workspace_bytes, void* stream);

/* out[m, n] = bf16( (float(sum_k a*b) * sa[m]) * sb[n] (+ bias[n]) ), int32 accumulation.
 * Replaces `robotics_integer::gemm` / `gemm_biasless` (ampere_ada/csrc/integer_gemm.cu:22-195).
 *   bits 8: a int8 [m, kpad], b int8 [n, kpad].  bits 4: packed nibbles [., kpad/2]; the kernel
 *   widens both operands to int8 in shared memory (tcgen05 has no 4-bit integer kind; products and
 *   int32 sums are identical), so W4A4 needs no scratch beyond the workspace header.
 *   sa f32 [m], sb f32 [n], bias bf16 [n] or NULL; out bf16 [m, n] contiguous;
 *   kpad % 128 == 0, n % 8 == 0; tactic 0..7 is accepted and never changes the result. */
int rk_gemm_int(const void* a, const float* sa, const void* b, const float* sb, const void* bias, void* out,
                int64_t m, int64_t n, int64_t kpad, int bits, int tactic, void* workspace,
                size_t workspace_bytes, void* stream);
/* rk_gemm_int with the residual update of a decoder layer applied in the epilogue, so that the
 * projection (o_proj, down_proj) writes the new residual stream itself:
 *   out[r, c] = bf16( residual[r, c] + t ),  t = y  (gate == NULL)  or  bf16( y * gate[r / tokens, c] ),
 * y = the bf16 value rk_gemm_int stores for the same arguments.  The arithmetic - and its three
 * roundings - is that of the tensor ops `x + y` / `x + y * gate` of the reference
 * (common/fused.py:47-58, models/pi05/modeling_gemma.py:226-244), i.e. of a projection followed by
 * the residual kernels; it equals handing (y, gate) to rk_gated_rmsnorm_quant_rows bit for bit.
 *   residual bf16 [m, n] contiguous; gate bf16 [m / tokens, n] contiguous or NULL; m % tokens == 0;
 *   out must not overlap residual.  One CTA per tile (no CTA-pair schedule). */
int rk_gemm_int_residual(const void* a, const float* sa, const void* b, const float* sb, const void* bias,
                         const void* residual, const void* gate, int64_t tokens, void* out, int64_t m, int64_t n,
                         int64_t kpad, int bits, int tactic, void* workspace, size_t workspace_bytes, void* stream);

/* Same product, but writes the raw int32 accumulators [m, n] (parity aid; no reference counterpart). */
int rk_gemm_int_acc(const void* a, const void* b, int32_t* acc, int64_t m, int64_t n, int64_t kpad, int bits,
                    int tactic, void* workspace, size_t workspace_bytes, void* stream);

/* W4A4 GEMM (the bits = 4 case of rk_gemm_int) for callers that cannot allocate device memory
 * when they call: code that runs inside a fixed memory plan, or a host thread that must stay out
 * of the allocator.  It has no counterpart in the reference.  The int8 copies of both operands,
 * which rk_gemm_int places in the caller's workspace, go to a device array built into the library
 * (8 MiB + 4 KiB; every GPU that loads the library holds it until the process exits), so there is
 * no workspace argument and nothing is allocated or freed, here or in any routine it calls.
 *   Limit: rk_workspace_bytes(RK_OP_W4A4, m, n, kpad) = 256 + round_up(m + n, 16) * kpad, rounded up
 *   to 256, must not exceed 8 MiB + 4 KiB; otherwise RK_EUNSUPPORTED (use rk_gemm_int instead).
 *   The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *   that first call outside any stream capture.
 *   All calls on a device share the one array: calls that may overlap on the GPU (different
 *   streams, or graphs replayed concurrently) race and must be serialised by the caller.
 *   The head of the array holds the device status word; it is cleared at the start of each call
 *   and read with rk_read_status(NULL, ...).
 * Arguments as rk_gemm_int with bits = 4. */
int rk_gemm_int4_noalloc(const void* a, const float* sa, const void* b, const float* sb, const void* bias,
                         void* out, int64_t m, int64_t n, int64_t kpad, int tactic, void* stream);

/* ---- W4A16 int4, group 128 -------------------------------------------------------------- */

/* Group-wise symmetric int4 weight packing: per (row, 128 consecutive k): s = bf16(max|w| / 7)
 * (1.0 when zero), q = clamp(rint(w / s), -7, 7) as a two's-complement nibble.  q uint8 [n, k/2];
 * scales bf16 [k/128, n].  Quantisation rules follow the reference's int4 packing
 * (ampere_ada/integer.py:250-263) and its mixed scale orientation
 * (blackwell/csrc/fp4_mixed_cutlass_linear.cu:89-90); k % 128 == 0.
 * Nibble order (this format's own, chosen for the GEMM's expansion step): eight consecutive
 * weights k0..k7 of a row occupy four bytes, byte b = k_b | (k_{b+4} << 4).  The packed buffer is
 * only meaningful to rk_gemm_w4a16_g128. */
int rk_pack_w4_g128(const void* w, int64_t n, int64_t k, void* q, void* scales, void* stream);
/* out[m, n] = bf16( sum_g s[g, n] * sum_{k in g} x[m, k] * q[n, k] (+ bias[n]) ), fp32 accumulation.
 * Stands in for `linear_w4a16` (blackwell/csrc/fp4_mixed_cutlass_linear.cu:190-410) with the
 * int4 / group-128 format.  x bf16 [m, k] contiguous, out bf16 [m, n] contiguous.
 *   m == 1 with tactic 0 and k in {1024, 2048, 4096, multiples of 8192}: a weight-streaming kernel
 *   on the CUDA cores (fp32 sums of exactly recovered x * q products; any tactic bit selects the
 *   tensor-core kernels instead).
 *   m <= 64: every group's sum is scaled in fp32 exactly as written above.  m > 64: the scale is
 *   folded into the expanded weight first, bf16(q * s) - one extra rounding of at most 2^-9 per
 *   weight, the order of operations of the reference's mixed-input GEMM; still within the 1e-2
 *   relative Frobenius bound of this operator.  tactic bit 1 (value 2) keeps the m <= 64
 *   arithmetic for any m; bit 0 selects four instead of eight expansion warps; bit 2 halves the
 *   activation tile; bit 3 (value 8) runs m > 128 on CTA pairs (`cta_group::2`), each CTA staging half of the
 *   activation tile; for m <= 32 sixteen expansion warps are used when
 *   k <= 4096: bit 4 (value 16) forces sixteen, bit 5 (value 32) forces eight.
 *   k % 128 == 0, n % 8 == 0, out 16-byte aligned. */
int rk_gemm_w4a16_g128(const void* x, const void* q, const void* scales, const void* bias, void* out,
                       int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                       void* stream);

/* ---- per-tensor FP8 --------------------------------------------------------------------- */

/* scale = max(max|x| / 448, 1e-12) over finite values; q = e4m3(clamp(x * (1/scale), +-448)).
 * Replaces `quantize_bf16` (blackwell/csrc/fp8_cutlass_linear.cu:61-101, 391-424).
 *   x bf16 [elements]; q e4m3 [elements]; scale_out f32 [1]; needs a workspace (header only). */
int rk_quant_tensor_fp8(const void* x, int64_t elements, void* q, float* scale_out, void* workspace,
                        size_t workspace_bytes, void* stream);
/* Same conversion with a caller-supplied scale.  Replaces `quantize_bf16_with_scale` (:885-911). */
int rk_quant_tensor_fp8_with_scale(const void* x, int64_t elements, const float* scale, void* q, void* stream);
/* out[m, n] = bf16( (scale_a * scale_b) * sum_k a*b (+ bias[n]) ), fp32 accumulation.
 * Replaces `linear_forward_packed` / `fp8_gemm::run` (blackwell/csrc/fp8_cutlass_linear.cu:473-723, 1026-1154).
 *   a e4m3 [m, k], b e4m3 [n, k]; scale_a, scale_b: device pointers to one f32; k % 16 == 0, n % 8 == 0. */
int rk_gemm_fp8(const void* a, const float* scale_a, const void* b, const float* scale_b, const void* bias,
                void* out, int64_t m, int64_t n, int64_t k, int tactic, void* workspace,
                size_t workspace_bytes, void* stream);

/* (residual add +) RMSNorm in front of the per-tensor quantizer.  s = bf16(x + residual) (s = x
 * when residual is NULL), r = rsqrt(mean(s^2) + eps), y = bf16( bf16(s * r) * weight[k] ); then
 * scale and codes as rk_quant_tensor_fp8 over y.  Replaces `add_rms_norm_quantize_bf16`
 * (blackwell/csrc/fp8_cutlass_linear.cu:145-269, 913-960).
 *   x, residual bf16 [rows, k]; weight bf16 [k]; sum_out bf16 [rows, k] or NULL (written only
 *   with a residual); norm_out bf16 [rows, k] (required); q e4m3 [rows, k]; scale_out f32 [1];
 *   k % 16 == 0, k <= 8192; needs a workspace (header only). */
int rk_rmsnorm_quant_fp8(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k,
                         float eps, void* sum_out, void* norm_out, void* q, float* scale_out, void* workspace,
                         size_t workspace_bytes, void* stream);
/* SwiGLU in front of the per-tensor quantizer: a = bf16( gate / (1 + exp(-gate)) * up ) in fp32,
 * gate = gate_up[r, 0:inter], up = gate_up[r, inter:2*inter]; scale = *scale_in when given, else
 * computed over a and written to scale_out.  Replaces `quantize_swiglu_bf16` and
 * `quantize_swiglu_bf16_with_scale` (blackwell/csrc/fp8_cutlass_linear.cu:271-389, 962-1009).
 *   gate_up bf16 [rows, 2*inter]; q e4m3 [rows, inter]; inter % 16 == 0. */
int rk_swiglu_quant_fp8(const void* gate_up, int64_t rows, int64_t inter, const float* scale_in, void* q,
                        float* scale_out, void* workspace, size_t workspace_bytes, void* stream);

/* The "producer" form of the FP8 GEMM: bf16 activations with a UNIT activation scale are converted
 * to e4m3 (clamped to +-448) inside the kernel - raw bf16 rows land in shared memory by TMA and
 * four warps rewrite them into the MMA's operand tile - so no e4m3 copy of the activations ever
 * exists in global memory and there is no separate quantizer launch.
 * out[m, n] = bf16( scale_b * sum_k e4m3(x) * b (+ bias[n]) ).  Replaces `linear_forward_producer` /
 * `fp8_producer_gemm::run` (blackwell/csrc/fp8_cutlass_linear.cu:727-856, 1268-1315).
 *   x bf16 [m, k] contiguous; b e4m3 [n, k]; scale_b: device pointer to one f32; k % 16 == 0, n % 8 == 0. */
int rk_gemm_fp8_producer(const void* x, const void* b, const float* scale_b, const void* bias, void* out,
                         int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                         void* stream);

/* ---- column-parallel FP8 linear with the exchange fused into the GEMM -------------------------
 *
 * Every GPU of a group of `ranks` holds the full [m, ld_total] bf16 output; rank r computes the
 * columns [col0, col0 + n_local) (its rows of the weight matrix) and the GEMM's epilogue stores
 * each finished 128 x 64 chunk straight into EVERY rank's buffer (TMA stores through peer
 * mappings; nothing is loaded from a peer).  When all stores of the launch have completed it
 * increments this rank's call counter (`epoch_counter`, one int32 of device memory, zero at the
 * start) and writes the new value to flag[rank] in every rank's flag array, its own included.
 * `rk_wait_peers` is the consumer side: a one-warp kernel on the caller's stream that counts its
 * own calls (`wait_counter`, another int32 of device memory, zero at the start) and returns once
 * every rank's flag - this rank's own too - has reached that count, or records device code 107 in
 * the workspace status word after about a second.  It is launched as a programmatic dependent: it
 * may start while the GEMM still runs, and the kernel launched after it is held until it returns.
 * Together they stand in for `linear_forward_packed` (blackwell/fp8_linear.py:66-100) followed by an
 * all-gather of the ranks' slabs, without a collective launch (the reference runs its linears on
 * one GPU; the split along the output channels is the multi-GPU mode this library adds for the
 * widest projections).  Both counters live on the device, so the calls can be captured in a
 * CUDA graph and replayed.  The caller owns the rendezvous: every rank makes the same sequence of
 * calls (one wait per GEMM), the buffer addresses are exchanged beforehand, and consecutive calls
 * alternate between two output buffers so that a fast rank never overwrites a buffer that a slow
 * rank still reads (a graph therefore holds an even number of calls).
 *
 * The stores take one of two routes.  TMA stores through peer mappings: `out_ptrs[g]` is rank g's
 * [m, ld_total] buffer as mapped on this GPU (this rank's own at g = rank); the slab crosses this
 * GPU's links ranks - 1 times and the rank's own copy stays local.  Or `multimem.st` to
 * `multicast_out`, the multicast address of the output buffers (an NVSwitch multicast object bound
 * to every rank's buffer, e.g. from torch's symmetric memory): one copy of the slab leaves this GPU
 * and the switch delivers it to every rank, this one included.
 *   a e4m3 [m, k]; b e4m3 [n_local, k] (this rank's rows of the weight); scales: device pointers to
 *   one f32 each (the activation scale must be the same on every rank); bias bf16 [n_local] or NULL;
 *   exactly one of out_ptrs / multicast_out is given; col0, n_local, ld_total multiples of 8;
 *   flag_ptrs[g]: rank g's int32 flag array [ranks] as mapped on this GPU. */
int rk_gemm_fp8_column_parallel(const void* a, const float* scale_a, const void* b, const float* scale_b,
                                const void* bias, int64_t m, int64_t n_local, int64_t k, void* const* out_ptrs,
                                void* multicast_out, int64_t ld_total, int64_t col0, void* const* flag_ptrs, int rank,
                                int ranks, void* epoch_counter, void* workspace, size_t workspace_bytes, void* stream);
/*   flags: this rank's own flag array [ranks]; wait_counter: one int32 of device memory owned by the waits. */
int rk_wait_peers(const void* flags, int ranks, void* wait_counter, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Exchange memory for the calls above: device memory that the other processes of the node map.
 * rk_peer_alloc: cudaMalloc of `bytes` (zero-filled) on the current device plus its 64-byte
 * inter-process handle.  rk_peer_open: maps another process's allocation (its handle and the
 * index of the device that owns it) with the CURRENT device, so that kernels on the current
 * device may store into it; fails with RK_EUNSUPPORTED when the two devices have no peer path.
 * rk_peer_close / rk_peer_free undo the two.  These four are set-up calls: they are the only
 * entry points that allocate or map device memory, and they synchronize the device. */
int rk_peer_alloc(size_t bytes, void** ptr, void* handle64);
int rk_peer_open(const void* handle64, int owner_device, void** ptr);
int rk_peer_close(void* ptr);
int rk_peer_free(void* ptr);

/* ---- MXFP8 ------------------------------------------------------------------------------ */

/* Per 32 consecutive k: SF = UE8M0 round-up of max|x| * rcp(448) (255 when the block holds a
 * non-finite value), q = e4m3(x * 2^-(SF-127)).  Replaces `robotics_mxfp8::pack`
 * (blackwell/csrc/mxfp8_cutlass_linear.cu:31-105).  x bf16 [rows, k], k % 32 == 0;
 * q e4m3 [rows, k]; sf: rk_sf_bytes(rows, k/32) bytes, fully written (padding = 0). */
int rk_pack_mxfp8(const void* x, int64_t rows, int64_t k, void* q, void* sf, void* stream);
/* SwiGLU producer for MXFP8: bf16( table[gate] * up ) packed like rk_pack_mxfp8, `table` = SiLU evaluated on
 * all 65536 bf16 bit patterns.  Replaces `robotics_mxfp8_swiglu::silu_mul_pack`
 * (blackwell/csrc/mxfp8_swiglu.cu:20-117, blackwell/mxfp8_swiglu.py:43-60).
 *   gate_up bf16 [rows, 2 * inter] contiguous, gate first; inter % 32 == 0;
 *   q e4m3 [rows, inter]; sf rk_sf_bytes(rows, inter / 32) bytes, every byte written. */
int rk_swiglu_pack_mxfp8(const void* gate_up, int64_t rows, int64_t inter, const void* silu_table, void* q, void* sf,
                         void* stream);

/* out = bf16( sum over blocks (sfa * sfb * sum_k a*b) (+ bias[n]) ).  Replaces `robotics_mxfp8::linear`
 * (blackwell/csrc/mxfp8_cutlass_linear.cu:107-258).  k % 32 == 0, n % 8 == 0. */
int rk_gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, const void* bias, void* out,
                  int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes,
                  void* stream);

/* ---- NVFP4 ------------------------------------------------------------------------------ */

/* Per 16 consecutive k: s = max|v| / 6 (1.0 when zero), SF = UE4M3(s), q = e2m1(v / float(SF)),
 * sixteen codes per 64-bit word, low nibble first; v = x, or x / *global_scale when
 * global_scale is not NULL.  Replaces `pack_linear_weight_gemm_bf16` / `pack_activation_gemm_bf16`
 * (blackwell/csrc/fp4_cutlass_linear.cu:789-841, 1530-1587).  x bf16 [rows, k], k % 32 == 0;
 * q uint8 [rows, k/2]; sf: rk_sf_bytes(rows, k/16) bytes, fully written. */
int rk_pack_nvfp4(const void* x, int64_t rows, int64_t k, const float* global_scale, void* q, void* sf,
                  void* stream);
/* (residual add +) RMSNorm packed straight to NVFP4 (values never leave the chip between the norm
 * and the packer).  Norm arithmetic as rk_rmsnorm_quant_fp8, block arithmetic as rk_pack_nvfp4
 * without a per-tensor scale.  Replaces `add_rms_norm_fp4_quant_bf16`
 * (blackwell/csrc/fp4_cutlass_linear.cu:843-929, 2538-2608).  sum_out, norm_out: bf16 [rows, k] or
 * NULL; q uint8 [rows, k/2]; sf: rk_sf_bytes(rows, k/16) bytes, fully written; k % 32 == 0, k <= 8192. */
int rk_rmsnorm_pack_nvfp4(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k,
                          float eps, void* sum_out, void* norm_out, void* q, void* sf, void* stream);
/* The producers of the two entry points above on their own: (residual add +) RMSNorm with bf16 rounding
 * after `* inv` and after `* weight` -> bf16 (`robotics_cutlass_fp4::rms_norm_bf16`, `add_rms_norm_bf16`,
 * blackwell/csrc/fp4_cutlass_linear.cu:429-476,2472-2536); k % 16 == 0; with a residual, sum_out receives
 * bf16(x + residual).  And SwiGLU in the reference's bf16x2 steps -> bf16 [rows, inter]
 * (`silu_mul_bf16`, :944-995,1988-2043), gate_up [rows, 2 * inter] in the plain or the 64-column
 * interleaved layout; inter % 8 == 0. */
int rk_rmsnorm_bf16(const void* x, const void* residual, const void* weight, int64_t rows, int64_t k, float eps,
                    void* sum_out, void* norm_out, void* stream);
int rk_silu_mul_bf16(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* out, void* stream);

/* SwiGLU packed straight to NVFP4: a = gate * rcp(1 + exp(-gate)) * up with every step rounded to
 * bf16 (the reference evaluates it in packed bf16 arithmetic), then blocks as rk_pack_nvfp4.
 * Replaces the packing half of `linear_forward_swiglu_gemm_bf16`
 * (blackwell/csrc/fp4_cutlass_linear.cu:997-1143), non-interleaved gate/up layout.
 *   gate_up bf16 [rows, 2*inter]; q uint8 [rows, inter/2]; sf: rk_sf_bytes(rows, inter/16); inter % 32 == 0. */
int rk_swiglu_pack_nvfp4(const void* gate_up, int64_t rows, int64_t inter, void* q, void* sf, void* stream);
/* *scale_out = max(max|x| / (6 * 448), 1e-12): the optional fp32 per-tensor scale of an NVFP4
 * tensor (absent from the reference, where alpha = 1: blackwell/csrc/fp4_cutlass_linear.cu:1358). */
int rk_nvfp4_global_scale(const void* x, int64_t elements, float* scale_out, void* workspace,
                          size_t workspace_bytes, void* stream);
/* out = bf16( alpha * sum over blocks (sfa * sfb * sum_k a*b) (+ bias[n]) ), alpha = *ga * *gb
 * (each NULL = 1).  Replaces `linear_forward_packed_gemm_bf16` / `gemm_bf16::run`
 * (blackwell/csrc/fp4_cutlass_linear.cu:1199-1447, 1751-1848).  k % 64 == 0, n % 8 == 0. */
int rk_gemm_nvfp4(const void* a, const void* sfa, const float* ga, const void* b, const void* sfb,
                  const float* gb, const void* bias, void* out, int64_t m, int64_t n, int64_t k, int tactic,
                  void* workspace, size_t workspace_bytes, void* stream);

/* The gate/up projection of a SwiGLU MLP in NVFP4 with the activation fused into the GEMM: the
 * weight rows are stored in the 64-row interleaved order (of every 128 rows the first 64 belong to
 * `up`, the next 64 to the matching `gate` channels), so one output tile holds both factors of 64
 * channels.  The epilogue forms silu(gate) * up - the two-launch path's arithmetic step for step:
 * bf16(alpha * acc), SwiGLU in bf16 steps - and packs it to NVFP4: the [m, n] bf16 intermediate
 * never exists.  Runs on CTA pairs (`tcgen05.mma.cta_group::2`) for every m.  The computation of
 * `Sm100BlockScaledPersistentDenseGemmSwigluFusionKernel` (blackwell/cute_fp4_swiglu_kernel.py:75-2629;
 * wrapper `cutlass_swiglu_fp4_packed`, blackwell/cute_fp4_swiglu.py:186-282) without its multicast
 * loads, and of `linear_forward_swiglu_gemm_bf16`'s producer half (blackwell/csrc/fp4_cutlass_linear.cu:997-1143).
 *   a, sfa, ga / b_interleaved [n, k/2], sfb, gb as for rk_gemm_nvfp4; n = 2 * intermediate size, n % 128 == 0;
 *   q_out uint8 [m, n/4]; sf_out rk_sf_bytes(m, n/32) bytes (every byte of the 128-row blocks is written). */
int rk_gemm_nvfp4_swiglu(const void* a, const void* sfa, const float* ga, const void* b_interleaved, const void* sfb,
                         const float* gb, void* q_out, void* sf_out, int64_t m, int64_t n, int64_t k, int tactic,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Gate/up projection in NVFP4 (operands as for rk_gemm_nvfp4_swiglu: weight rows interleaved in blocks of 64, up
 * rows then their gate rows) whose epilogue writes the gated activation bf16( table[gate] * up ) - `table` a
 * 65536-entry bf16 table of the activation function, the arithmetic of rk_lut_mul_tensor_scale - as a bf16
 * matrix [m, n / 2] and, when scale_out is given, max(amax(out) / divisor, 1e-12): the GELU-gated MLP of the
 * Gemma layers (models/pi05/modeling_gemma.py:115-128) in front of a per-tensor-scaled packer, without the
 * [m, n] bf16 gate/up tensor.  Bit for bit rk_gemm_nvfp4 on the interleaved weight followed by
 * rk_lut_mul_tensor_scale on the de-interleaved result.  Needs a workspace header. */
int rk_gemm_nvfp4_gated_act(const void* a, const void* sfa, const float* ga, const void* b_interleaved, const void* sfb,
                            const float* gb, const void* table, float divisor, void* out, float* scale_out, int64_t m,
                            int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes, void* stream);

/* The MXFP8 sibling: gate/up projection in MXFP8 (operands as for rk_gemm_mxfp8, weight rows interleaved in blocks
 * of 64: up rows, then their gate rows) whose epilogue applies the table-SiLU SwiGLU producer and packs the
 * activation to MXFP8 - bit for bit rk_gemm_mxfp8 -> bf16 -> rk_swiglu_pack_mxfp8 on the de-interleaved result.
 * Replaces `cute_mxfp8_swiglu.cutlass_swiglu_mxfp8_packed` (blackwell/cute_mxfp8_swiglu.py:138-224; the CuTe-DSL
 * kernel's multicast loads are not restated).
 *   n = 2 * inter, n % 256 == 0; q_out e4m3 [m, inter]; sf_out rk_sf_bytes(m, inter / 32) bytes, every byte of
 *   the blocks of 128 rows that hold rows < m written; silu_table bf16 [65536]. */
int rk_gemm_mxfp8_swiglu(const void* a, const void* sfa, const void* b_interleaved, const void* sfb, const void* silu_table,
                         void* q_out, void* sf_out, int64_t m, int64_t n, int64_t k, int tactic, void* workspace,
                         size_t workspace_bytes, void* stream);

/* The same with a choice of gate/up layout: interleaved != 0 reads blocks of 128 columns holding 64 up
 * values followed by their 64 gate values (the layout of a fused gate/up projection,
 * blackwell/csrc/fp4_cutlass_linear.cu:958-965, 1051-1143); inter % 64 == 0 then. */
int rk_swiglu_pack_nvfp4_layout(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* q, void* sf,
                                void* stream);

/* ---- W4A8 MX: MXFP4 weights x MXFP8 activations ------------------------------------------------ */

/* Per 32 consecutive k: s = the smallest power of two >= max|w| / 6 (1.0 for a zero block), stored as
 * a UE8M0 byte; q = e2m1(w / s), two codes per byte, low nibble = even k.  Replaces `pack_mxfp4_weight`
 * (blackwell/csrc/fp4_mx_cutlass_linear.cu:59-100).  w bf16 [rows, k], k % 32 == 0; q uint8 [rows, k/2];
 * sf: rk_sf_bytes(rows, k/32) bytes, fully written. */
int rk_pack_mxfp4_weight(const void* w, int64_t rows, int64_t k, void* q, void* sf, void* stream);
/* Per 32 consecutive k: s = the smallest power of two >= max|x| / 448; q = e4m3(clamp(x / s, +-448)).
 * Replaces `pack_mxfp8_activation` (blackwell/csrc/fp4_mx_cutlass_linear.cu:103-132).  (The MXFP8 GEMM's
 * own packer, rk_pack_mxfp8, rounds max|x| * rcp(448) up instead and marks non-finite blocks.) */
int rk_pack_mxfp8_act_w4a8(const void* x, int64_t rows, int64_t k, void* q, void* sf, void* stream);
/* SwiGLU in front of the same block quantizer: a = gate / (1 + exp(-gate)) * up in fp32 (not rounded
 * to bf16).  Replaces `pack_swiglu_mxfp8` (blackwell/csrc/fp4_mx_cutlass_linear.cu:134-179).
 *   gate_up bf16 [rows, 2*inter] (gate first, or the interleaved layout above); q e4m3 [rows, inter]. */
int rk_swiglu_pack_mxfp8_w4a8(const void* gate_up, int64_t rows, int64_t inter, int interleaved, void* q, void* sf,
                              void* stream);
/* out = bf16( sum over 32-blocks (sfa * sfb * sum_k a*b) (+ bias[n]) ): MXFP8 activations against MXFP4
 * weights.  The packed weights are expanded to e4m3 (which holds every e2m1 value exactly) in shared
 * memory and the product runs as kind::mxf8f6f4 with both UE8M0 scale sets.  Replaces
 * `linear_w4a8_packed` / `mx_gemm::run` / `mx_swap_gemm::run` (blackwell/csrc/fp4_mx_cutlass_linear.cu:285-555).
 *   a e4m3 [m, k], sfa rk_sf_bytes(m, k/32); b uint8 [n, k/2], sfb rk_sf_bytes(n, k/32); k % 32 == 0, n % 8 == 0. */
int rk_gemm_w4a8_mx(const void* a, const void* sfa, const void* b, const void* sfb, const void* bias, void* out,
                    int64_t m, int64_t n, int64_t k, int tactic, void* workspace, size_t workspace_bytes, void* stream);

/* ---- between the q/k/v projection and attention ------------------------------------------- */
/* Rotary embedding of fresh query / key rows fused with the key / value cache update: one launch
 * instead of the ~14 tensor ops of apply_rotary_pos_emb + transposes + concatenation
 * (models/pi05/modeling_gemma.py:178-209, 247-274).  Stands in for `fused_cache_update_rope_bf16`
 * (blackwell/csrc/fp4_cutlass_linear.cu:478-588, arithmetic of rope_element :96-126) for caches that
 * are preallocated and already hold the prefix: only rows [prefix, prefix + tokens) are written.
 *   out = bf16( bf16(x * cos) + bf16(r * sin) ), r = -x[j + d/2] (j < d/2) or x[j - d/2].
 *   q bf16 rows [batch*tokens] of heads*head_dim elements, row stride q_stride elements (likewise
 *   k, v with kv_heads); q, k, v may be slices of one projection output.  cos, sin bf16
 *   [batch, tokens, head_dim]; q_out bf16 [batch, heads, tokens, head_dim], or - q_token_major != 0 -
 *   [batch, tokens, heads, head_dim] (the layout fused attention kernels read without a copy);
 *   k_cache, v_cache bf16
 *   [batch, kv_heads, cache_rows, head_dim].  head_dim % 16 == 0, <= 512; strides % 8 == 0; all
 *   pointers 16-byte aligned. */
int rk_rope_cache_update(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                         int64_t v_stride, const void* cos, const void* sin, int64_t batch, int64_t tokens,
                         int64_t heads, int64_t kv_heads, int64_t head_dim, void* q_out, int q_token_major,
                         void* k_cache, void* v_cache, int64_t cache_rows, int64_t prefix, void* stream);

/* The same, additionally writing the fresh value rows into a TRANSPOSED value cache
 * vt_cache bf16 [batch, kv_heads, head_dim, vt_pitch] (column prefix + token), which is the layout
 * rk_attention_prefix reads.  vt_pitch >= prefix + tokens. */
int rk_rope_cache_update_vt(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                            int64_t v_stride, const void* cos, const void* sin, int64_t batch, int64_t tokens,
                            int64_t heads, int64_t kv_heads, int64_t head_dim, void* q_out, int q_token_major,
                            void* k_cache, void* v_cache, int64_t cache_rows, int64_t prefix, void* vt_cache,
                            int64_t vt_pitch, void* stream);

/* Attention of `tokens` fresh query tokens per sequence over kv_len cached keys / values (all keys
 * visible to all queries), grouped-query.  Stands in for the eager attention of the action expert
 * (models/pi05/modeling_gemma.py:247-274) with its arithmetic: scores = bf16(q . k) * scaling in
 * bf16, softmax in fp32 over all keys, probabilities rounded to bf16, output = bf16 of the fp32 sum
 * of p * v.  One launch: QK^T and PV on the tensor cores, keys split over a thread-block cluster
 * whose CTAs exchange the softmax statistics and sum their partial outputs on chip.
 *   q bf16 [batch, tokens, heads, 256] (the token-major output of rk_rope_cache_update);
 *   k_cache bf16 [batch, kv_heads, cache_rows, 256]; vt_cache bf16 [batch, kv_heads, 256, vt_pitch]
 *   (values transposed; columns at and beyond kv_len must hold finite numbers, e.g. zeros);
 *   out bf16 [batch, tokens, heads, 256].  head_dim == 256; tokens <= 128; kv_len <= 2048,
 *   kv_len <= cache_rows, kv_len <= vt_pitch, vt_pitch % 8 == 0; heads % kv_heads == 0;
 *   needs a workspace (header only). */
int rk_attention_prefix(const void* q, const void* k_cache, const void* vt_cache, void* out, int64_t batch,
                        int64_t tokens, int64_t heads, int64_t kv_heads, int64_t head_dim, int64_t cache_rows,
                        int64_t vt_pitch, int64_t kv_len, float scaling, void* workspace, size_t workspace_bytes,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RK_B200_H_ */
