/*
 * dsb.h - C ABI of libdsb.so: the B200 (sm_100a) kernels behind the DiT
 * denoising step of DiffSynth-Engine (Flux / Wan2.1 / MMDiT double-stream
 * blocks).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless said
 *     otherwise; the library allocates nothing and never synchronises.
 *   - `stream` is a cudaStream_t passed as void*; kernels are enqueued on it.
 *   - Return value: 0 on success, a negative DSB_ERR_* code otherwise.  The
 *     functions never throw and never terminate the process.
 *   - `status` (where present) is an optional device int the kernel sets to
 *     DSB_ERR_TIMEOUT if one of its bounded on-chip waits ran out; it is never
 *     cleared by the library.
 *   - Leading dimensions (`ld_*`) are in ELEMENTS of the tensor they describe.
 *   - bf16 tensors need 16-byte aligned bases and leading dimensions that are
 *     multiples of 8 elements; 8-bit tensors need multiples of 16.
 *
 * Each entry point names the code of the reference (paths inside
 * modelscope/DiffSynth-Engine v0.1.1) whose arithmetic it replaces.
 */
#ifndef DSB_H_
#define DSB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSB_OK 0
#define DSB_ERR_ARG (-1)
#define DSB_ERR_CUDA (-2)
#define DSB_ERR_TIMEOUT (-3)
#define DSB_ERR_UNSUPPORTED (-4)
#define DSB_ERR_TOO_LARGE (-5) /* problem exceeds the fixed scratch of a *_static entry point */

/* element formats */
#define DSB_FMT_BF16 0
#define DSB_FMT_E4M3 1
#define DSB_FMT_INT8 2

/* epilogue activation */
#define DSB_ACT_NONE 0
#define DSB_ACT_GELU_TANH 1
#define DSB_ACT_SILU 2
#define DSB_ACT_GELU 3 /* exact (erf) GELU: torch.nn.GELU() of the Wan image-embedding MLP, wan_dit.py:208 */

/* Library/ABI version (major*100 + minor). */
int dsb_version(void);

/* Self-test of the bounded device waits (no counterpart in the reference, which has no device-side waits): a
 * one-CTA kernel in which one role waits, for at most `limit_cycles` SM cycles (<= 2e9), on a barrier nothing ever
 * arrives at, while a second role waits on the same barrier with the library's ordinary one-second budget.  The
 * first role gives up and raises the CTA's abort flag, the second sees the flag and leaves too (`*neighbour_left`
 * = 1), and `*status` becomes DSB_ERR_TIMEOUT - the sequence every kernel of this library follows when a wait of
 * its own runs out.  The context stays usable.  `status` must be 0 on entry to observe the result. */
int dsb_selftest_wait_timeout(long long limit_cycles, int* status, int* neighbour_left, void* stream);

/*
 * AdaLN: y = LayerNorm(x; eps, no affine) * (1 + scale[d]) + shift[d] over rows of width D.
 * out_fmt BF16 writes bf16; E4M3 / INT8 write the quantised operand of the next GEMM and
 * row_scale[m] = amax(row)/448 (or /127), y_q = round(y / row_scale).
 * Replaces: models/basic/transformer_helper.py:13-22,32-36 (AdaLayerNorm, AdaLayerNormSingle),
 * models/flux/flux_dit.py:228,233,331-335, models/wan/wan_dit.py:25-26,188,191 (modulate(norm(x))),
 * and, with scale = weight-1 / shift = bias, the affine LayerNorm models/wan/wan_dit.py:178,190.
 */
int dsb_ln_modulate(const void* x, int64_t ld_x, const float* shift, const float* scale, void* y, int64_t ld_y,
                    float* row_scale, int M, int D, float eps, int out_fmt, void* stream);

/*
 * dsb_ln_modulate with two modulation sets: rows [0, split_row) use (shift, scale), rows [split_row, M) use
 * (shift_b, scale_b) - the text rows and the image rows of the joint hidden-state buffer, each with its own AdaLN
 * output (models/flux/flux_dit.py:220-221,228,233), normalised in one launch.
 */
int dsb_ln_modulate2(const void* x, int64_t ld_x, const float* shift, const float* scale, int split_row,
                     const float* shift_b, const float* scale_b, void* y, int64_t ld_y, float* row_scale, int M, int D,
                     float eps, int out_fmt, void* stream);

/*
 * out = x + gate[d] * y (gate NULL: out = x + y); bf16 in/out, fp32 gate.
 * Replaces: models/flux/flux_dit.py:227,229,232,234,318-319; models/wan/wan_dit.py:189,190,192.
 */
int dsb_gate_residual(const void* x, int64_t ld_x, const void* y, int64_t ld_y, const float* gate, void* out,
                      int64_t ld_o, int M, int D, void* stream);

/*
 * In-place per-head RMSNorm (head_dim 128, fp32 weights w_q/w_k[128]) + RoPE on adjacent pairs for
 * the first nsel*H heads of each row of buf[S, ld] (nsel=2: q heads then k heads; nsel=1: q only).
 * rope: fp32 [rows, 64, 2] = (cos, sin) per pair, row (rope_row0 + s) for token s; NULL = no rotation.
 * Replaces: models/basic/transformer_helper.py:73-78 (RMSNorm) and models/flux/flux_dit.py:154-159 (apply_rope).
 */
int dsb_rmsnorm_rope_heads(void* buf, int64_t ld, int S, int H, int head_dim, int nsel, const float* w_q,
                           const float* w_k, const float* rope, int rope_row0, float eps, void* stream);

/*
 * RMSNorm over the whole row (width D = heads*128, fp32 weight w[D]) followed by per-head RoPE with the token's
 * 64 (cos, sin) pairs (rope NULL = none); out may equal x (in place).  With out_chunk_cols > 0 column c of row m is
 * written to out[(c / out_chunk_cols) * out_chunk_stride + m * ld_out + c % out_chunk_cols], i.e. straight into the
 * per-peer-contiguous send buffer [P][rows][D/P] of the sequence-parallel head exchange (0 = plain rows).
 * Replaces: models/wan/wan_dit.py:61-78 (RMSNorm over all heads) and :54-58 (rope_apply).
 */
int dsb_rmsnorm_full(const void* x, int64_t ld_x, void* out, int64_t ld_out, int out_chunk_cols,
                     int64_t out_chunk_stride, int M, int D, const float* w, const float* rope, int rope_row0,
                     float eps, void* stream);

/*
 * Dynamic per-row quantisation of a bf16 activation: y_q[m,:] = round(x[m,:] / s_m), s_m = amax/448 (E4M3,
 * round-to-nearest-even, saturating) or amax/127 (INT8, round-half-even); an all-zero row gets s_m = 1.
 * Replaces: the activation cast of utils/fp8_linear.py:35 (which uses unit scale).
 */
int dsb_quant_rows(const void* x, int64_t ld_x, void* y, int64_t ld_y, float* row_scale, int M, int K, int out_fmt,
                   void* stream);

/*
 * dsb_quant_rows reading a chunked activation: column c of row m is x[(c / chunk_cols) * chunk_stride + m * ld_x +
 * c % chunk_cols] - what the reverse head/sequence all-to-all delivers ([P][rows][K/P]); the output is plain rows.
 * No reference counterpart (the reference has no sequence parallelism); arithmetic as dsb_quant_rows.
 */
int dsb_quant_rows_chunked(const void* x, int64_t ld_x, int chunk_cols, int64_t chunk_stride, void* y, int64_t ld_y,
                           float* row_scale, int M, int K, int out_fmt, void* stream);

/*
 * GGUF Q8_0 -> bf16: blocks [N, row_bytes] of raw bytes (K/32 blocks of 34 bytes per row: fp16 d, 32 x int8 q; 2-byte
 * aligned), out[n, k] = bf16(bf16(d) * q), bit-identical to dequantize_blocks_Q8_0 with a bf16 compute dtype
 * (utils/gguf.py:171-175).  Meant to run ONCE per weight when a GGUF checkpoint is attached (the reference
 * dequantises the whole weight inside every Linear call, utils/gguf.py:77-84): with 180 GB of HBM the bf16 (or
 * re-quantised FP8/INT8) copy stays resident, and a compute-bound GEMM gains nothing from converting its operand on
 * every one of its M/128 passes over the weight.  K % 32 == 0.
 */
int dsb_dequant_q8_0(const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out, void* stream);

/*
 * GGUF Q4_K -> bf16, same role as dsb_dequant_q8_0: blocks [N, row_bytes] with K/256 super-blocks of 144 bytes per row
 * (16-byte aligned rows), out bit-identical to dequantize_blocks_Q4_K with a bf16 compute dtype
 * (utils/gguf.py:158-168,298-315), including its bf16 rounding after every product.  K % 256 == 0.
 */
int dsb_dequant_q4_k(const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out, void* stream);

/* Any GGUF block format the reference dequantises (utils/gguf.py:137-147 `dequantize_functions`, :171-368): Q4_0,
 * Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, named by ggml's type number (2, 3, 6, 7, 8, 10, 11, 12, 13,
 * 14).  raw rows `[N, K / block * bytes]` -> bf16 `[N, K]`, bit-identical to the reference's `dequantize` with bf16
 * as compute dtype (the same products and sums, each rounded to bf16).  K must be a multiple of the block size (32,
 * or 256 for the K-quants); `row_bytes` is the pitch of a raw row.  DSB_ERR_UNSUPPORTED for any other type. */
int dsb_dequant_gguf(int ggml_type, const void* blocks, int64_t row_bytes, int N, int K, void* out, int64_t ld_out,
                     void* stream);

/*
 * y = saturating cast of bf16 x [M, ld_x] (D columns, D % 8 == 0) to e4m3 (round-to-nearest-even, +-448) or int8
 * (round-half-even, +-127), no scale: the values are already in operand units.  y may be a column window of a wider
 * 8-bit buffer (ld_y in elements, 8-byte aligned start).  split != 0 (e4m3 only) writes three windows of D columns,
 * [head | remainder | head] with head = e4m3(x), remainder = e4m3(x - head).  Used to place the LoRA
 * down-projection next to the quantised activations so that the side matrices ride in the main GEMM as extra K
 * columns; replaces the separate up(down(x)) GEMMs and the scaled add of models/basic/lora.py:29-32,137-141.
 */
int dsb_cast_quant(const void* x, int64_t ld_x, void* y, int64_t ld_y, int M, int D, int out_fmt, int split,
                   void* stream);

/*
 * y[n] = act_out((sum_k W[n,k] * act_in(x[k])) * w_scale[n*w_scale_stride] + bias[n]) for one activation row
 * (fp32 x, fp32 y).  W is [N, ld_w] in w_fmt.  act_in: 0 none, DSB_ACT_SILU; act_out: DSB_ACT_*;
 * accumulate != 0 adds the result to y instead of overwriting it.
 * Replaces the M=1 Linears: models/basic/transformer_helper.py:14,33 and models/flux/flux_dit.py:332
 * (SiLU -> Linear of the AdaLN layers), models/basic/timestep.py:73-81, models/flux/flux_dit.py:348-352,
 * models/wan/wan_dit.py:279-287,327-328.
 */
int dsb_gemv(const void* W, int64_t ld_w, int w_fmt, const float* x, const float* w_scale, int w_scale_stride,
             const float* bias, float* y, int N, int K, int act_in, int act_out, int accumulate, void* stream);

/*
 * Sinusoidal timestep embedding of n scalars t[r] * t_scale into out[n, dim] = [cos | sin] (fp32, optionally
 * rounded to bf16 values as the reference casts to the model dtype).
 *   mode 0: fp32 angles, freq_i = exp(-ln(10000) i / (dim/2))   models/basic/timestep.py:6-44 (flip_sin_to_cos,
 *           downscale_freq_shift 0, as configured at :68-70)
 *   mode 1: fp64 angles, freq_i = 10000^(-i / (dim/2))          models/wan/wan_dit.py:29-35
 */
int dsb_timestep_embedding(const float* t, int n, int dim, float t_scale, int mode, int round_bf16, float* out,
                           void* stream);

/*
 * out = cast(latents + model_out * dt), optionally after the inpaint blend
 * model_out = model_out*mask + init*(1-mask).  is_f32 selects fp32 or bf16 tensors.
 * Replaces: algorithm/sampler/flow_match/flow_match_euler.py:11-19.
 */
int dsb_euler_step(const void* latents, const void* model_out, const void* init, const void* mask, float dt,
                   void* out, int64_t n, int is_f32, void* stream);

/*
 * Classifier-free-guidance combine fused with the sampler update:
 *   model_out = neg + cfg_scale * (pos - neg);   out = cast(latents + model_out * dt)
 * Replaces: pipelines/wan_video.py:230,248 and pipelines/flux_image.py:387,398 (noise_pred = negative + cfg_scale *
 * (positive - negative)) followed by algorithm/sampler/flow_match/flow_match_euler.py:11-19; bit-identical to that
 * tensor expression for bf16 (same rounding points) and fp32.
 */
int dsb_cfg_euler_step(const void* latents, const void* pos, const void* neg, float cfg_scale, float dt, void* out,
                       int64_t n, int is_f32, void* stream);

/*
 * Quantised / bf16 Linear on the tensor cores:
 *   acc[m,n]  = sum_k A[m,k] * W[n,k]                      (fp32 accumulate; int32 for INT8)
 *   v         = acc * row_scale[m] * col_scale[n*col_scale_stride] + bias[n]
 *   v         = act(v)            for columns n >= act_col0 (act = DSB_ACT_*)
 *   v         = resid[m,n] + gate[n] * v                    when resid != NULL (gate NULL = 1)
 *   out0[m,n] = bf16(v) for n < split_col, out1[m, n-split_col] = bf16(v) otherwise
 * A is [M, lda] and W is [N, ldw], both with K contiguous, in `fmt` (BF16, E4M3 or INT8).  row_scale,
 * col_scale, bias, gate, resid and out1 may be NULL (pass split_col >= N when out1 is unused; split_col
 * must be a multiple of 256).  K-tails and M/N-tails are handled; N and split_col must be multiples of 8.
 * Replaces: utils/fp8_linear.py:27-60 (cast + torch._scaled_mm + bias), the dequantise-then-F.linear of
 * utils/gguf.py:77-84, and the elementwise code the reference runs after each Linear:
 * GELU-tanh (models/flux/flux_dit.py:209,215,315; models/wan/wan_dit.py:180) and the gate-residual lines above.
 */
int dsb_gemm(const void* A, int64_t lda, const void* W, int64_t ldw, int fmt, int M, int N, int K,
             const float* row_scale, const float* col_scale, int col_scale_stride, const float* bias, int act,
             int act_col0, const float* gate, const void* resid, int64_t ld_resid, void* out0, int64_t ld_out0,
             void* out1, int64_t ld_out1, int split_col, int* status, void* stream);

/*
 * dsb_gemm for a fused q|k|v (|mlp) projection, with the per-head QK-RMSNorm and RoPE applied in the epilogue:
 * columns [0, d_model) are q heads (weights nq_w[128]), [d_model, 2 d_model) k heads (nk_w[128]); each head's 128
 * columns are scaled by rsqrt(mean(v^2) + norm_eps) * w and then rotated pairwise with rope[(rope_row0 + m)*64 + j]
 * = (cos, sin) (rope NULL: no rotation).  Here the table is FP16, [rows >= rope_row0 + M][64][2], 16-byte aligned:
 * the epilogue fetches it with TMA tile loads, 128 bytes per row and 64 output columns, like a residual block
 * (per-thread loads of an fp32 table cost the 4096x3072->9216 projection 40 % of its time).  fp16 cos/sin are
 * exact to 2^-12, an eighth of the bf16 rounding of the result.  Columns from 2 d_model on follow dsb_gemm (bias, activation from act_col0,
 * split output).  Replaces, on top of dsb_gemm: models/basic/transformer_helper.py:73-78 (RMSNorm) and
 * models/flux/flux_dit.py:154-159 (apply_rope) as used at flux_dit.py:165-180 and :297-301.
 */
int dsb_gemm_qkv(const void* A, int64_t lda, const void* W, int64_t ldw, int fmt, int M, int N, int K,
                 const float* row_scale, const float* col_scale, int col_scale_stride, const float* bias, int act,
                 int act_col0, void* out0, int64_t ld_out0, void* out1, int64_t ld_out1, int split_col,
                 const float* nq_w, const float* nk_w, int d_model, const void* rope, int rope_row0, float norm_eps,
                 int* status, void* stream);

/*
 * One problem of a grouped launch: the arguments of dsb_gemm / dsb_gemm_qkv as a struct (nq_w NULL = no fused
 * QK-RMSNorm/RoPE; resid NULL = no residual form; out1 NULL = one output).
 */
typedef struct dsb_gemm_args {
  const void* A; int64_t lda;
  const void* W; int64_t ldw;
  int M, N, K;
  const float* row_scale;
  const float* col_scale; int col_scale_stride;
  const float* bias;
  int act, act_col0;
  const float* gate;
  const void* resid; int64_t ld_resid;
  void* out0; int64_t ld_out0;
  void* out1; int64_t ld_out1;
  int split_col;
  const float* nq_w; const float* nk_w; int d_model;
  const void* rope; /* fp16 (cos, sin) table, see dsb_gemm_qkv */ int rope_row0; float norm_eps;
  /* DSB_FMT_BF16 (0) or DSB_FMT_E4M3: out0 / out1 written as e4m3 with unit scale (saturating cast of the fp32
   * epilogue value; ld in elements = bytes, multiple of 16), which is the reference's own activation rule
   * (utils/fp8_linear.py:35), so that the Linear consuming it needs no row quantiser.  Not with resid; normalised
   * head columns (nq_w) stay bf16. */
  int out0_fmt, out1_fmt;
} dsb_gemm_args;

/*
 * count (1 or 2) independent GEMMs of one format in ONE persistent launch: the tile list of the second problem
 * follows the first, so the 512-row text-stream Linear of a double-stream block runs on the SMs that the
 * 4096-row image-stream Linear leaves idle in its last wave (models/flux/flux_dit.py:165-174,189-193,229,234 issue
 * them one after the other).  Arithmetic per problem exactly as dsb_gemm / dsb_gemm_qkv; the tile shape is chosen
 * for args[0].
 */
int dsb_gemm_group(const dsb_gemm_args* args, int count, int fmt, int* status, void* stream);

/*
 * Attention without mask: o[b,s,h,:] = softmax(q[b,s,h,:] . k[b,:,h,:]^T * sm_scale) v[b,:,h,:], head_dim 128,
 * bf16 in/out, fp32 softmax statistics.  Tensors are addressed as base + b*stride_b + s*stride_s + h*stride_h
 * (+ d, contiguous); strides are in elements and need to be multiples of 8.  Covers the joint text+image
 * self-attention (Sq == Sk) and cross-attention (Sk = context length).
 * Replaces: the default of models/flux/flux_dit.py:21 (_attn_func, called at :182,:267,:303) and
 * models/wan/wan_dit.py:18-22 (attention).
 */
int dsb_flash_attn(const void* q, const void* k, const void* v, void* o, int B, int H, int Sq, int Sk, int head_dim,
                   int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h, int64_t k_stride_b,
                   int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s,
                   int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h, float sm_scale,
                   int* status, void* stream);

/*
 * dsb_flash_attn with the output written as e4m3 (1 byte per element, o strides in elements = bytes, multiples of 16):
 * the value is rounded to bf16 and then cast with saturation, bit for bit what dsb_flash_attn followed by
 * dsb_cast_quant (unit scale) produces - the activation rule of the reference's FP8 Linear (utils/fp8_linear.py:35)
 * applied by the producing kernel, for callers whose next op is an FP8 Linear (Flux single blocks,
 * models/flux/flux_dit.py:303-320).
 */
int dsb_flash_attn_out8(const void* q, const void* k, const void* v, void* o, int B, int H, int Sq, int Sk, int head_dim,
                        int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h, int64_t k_stride_b,
                        int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s,
                        int64_t v_stride_h, int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h, float sm_scale,
                        int* status, void* stream);

/*
 * dsb_flash_attn for one sample (B = 1) whose query rows and output rows are each cut into equal row ranges that live
 * in separate buffers: query rows [i*q_rows_per_part, (i+1)*q_rows_per_part) are read from q_parts[i] (addressed as
 * base + s*q_stride_s + h*q_stride_h with s counted from the start of the part; q_rows_per_part a multiple of 128;
 * every part holds q_rows_per_part rows, those past Sq are read and ignored),
 * output row s is written to o_parts[s / o_rows_per_part] at row s % o_rows_per_part.  The parts may be memory of
 * other GPUs that this process has mapped (peer access): the kernel then reads its queries from, and writes its
 * result to, the ranks that own those tokens - the all-to-all on both sides of the sequence-parallel attention of
 * utils/parallel.py's ParallelModel users (pipelines/wan_video.py:434-455) happens inside the attention kernel
 * (plain tiled TMA loads without multicast, plain stores).  q_parts / o_parts are host arrays of device pointers,
 * n_*_parts <= 8 each, n * rows_per_part >= Sq.
 * workspace (optional, device memory on the launching GPU, 16-byte aligned): when the (query-tile pair, head) items do
 * not fill the last wave of one CTA per SM, the items of that wave are cut along the keys into 2..4 CTAs each and a
 * small second kernel combines their partial results; needs tail_items * split * 256 * 528 bytes
 * (dsb_flash_attn_workspace_bytes gives the bound); without it, or if it is too small, nothing is cut.
 */
int dsb_flash_attn_parts(const void* const* q_parts, int n_q_parts, int q_rows_per_part, const void* k, const void* v,
                         void* const* o_parts, int n_o_parts, int o_rows_per_part, int H, int Sq, int Sk, int head_dim,
                         int64_t q_stride_s, int64_t q_stride_h, int64_t k_stride_s, int64_t k_stride_h,
                         int64_t v_stride_s, int64_t v_stride_h, int64_t o_stride_s, int64_t o_stride_h,
                         float sm_scale, void* workspace, int64_t workspace_bytes, int* status, void* stream);

/* Upper bound of the workspace dsb_flash_attn_parts can use on the current device (a last wave of sm_count - 1 items
 * cut in four: 80 MB on a 148-SM part). */
int64_t dsb_flash_attn_workspace_bytes(void);

/*
 * Barrier among the n_ranks (<= 8) GPUs of a sequence-parallel group, launched by every rank on its own stream:
 * flags[r] points to rank r's array of n_ranks ints (zero before the first barrier) in memory all ranks have mapped;
 * epoch must grow by one per barrier.  Everything this rank's earlier launches on the stream wrote, to any rank's
 * memory, is visible to the launches that follow the barrier on every other rank.  A rank that does not arrive within
 * limit_cycles SM cycles makes the waiters return with *status = DSB_ERR_TIMEOUT (no trap, the context stays usable);
 * while *status is non-zero later barriers signal but do not wait.
 * Stands where the reference's wrappers synchronise ranks through torch.distributed collectives
 * (utils/parallel.py:112-135).
 */
int dsb_rank_barrier(int* const* flags, int n_ranks, int rank, int epoch, long long limit_cycles, int* status,
                     void* stream);

/*
 * Patch embedding input: latents [C, F, 2*gh, 2*gw] (bf16, contiguous) -> rows [n_rows, ld_out] for tokens
 * row0 .. row0+n_rows-1 in (f, y, z) raster order, feature c*4 + py*2 + pz (C <= 128); rows past the last token are
 * zeros.  out_fmt BF16 writes bf16; E4M3 / INT8 write the row quantised with its dynamic per-row scale (the rule of
 * dsb_quant_rows) into row_scale[n_rows], so the row quantiser in front of the patch-embedding GEMM disappears.
 * Replaces: the strided gather of WanDiT.patchify's Conv3d (models/wan/wan_dit.py:271-273,301-305) and
 * FluxDiT.patchify (models/flux/flux_dit.py:364-367).
 */
int dsb_patchify(const void* latents, int C, int F, int gh, int gw, int row0, int n_rows, int out_fmt, void* out,
                 int64_t ld_out, float* row_scale, void* stream);

/*
 * Token rows [F*gh*gw, ld_tok] (bf16, >= C*4 features) -> latents [C, F, 2*gh, 2*gw].  c_fastest 1: feature
 * (py*2 + pz)*C + c (WanDiT.unpatchify, models/wan/wan_dit.py:307-317); 0: feature c*4 + py*2 + pz
 * (FluxDiT.unpatchify, models/flux/flux_dit.py:369-374).
 */
int dsb_unpatchify(const void* tokens, int64_t ld_tok, int C, int F, int gh, int gw, int c_fastest, void* out,
                   void* stream);

/*
 * Weight prepack: W[N,K] (fp32 or bf16 by src_is_bf16) -> quantised payload [N,K] row-major plus scales.
 *   fmt E4M3, per_channel 0: s = amax(|W|)/448 (one scale);   per_channel 1: s_n = amax(|W[n,:]|)/448
 *   fmt INT8 (per_channel 1 only): s_n = amax/127, q = round-half-even(W/s) clamped to +-127
 * scales receives 1 or N floats.  `work` is a device float (scratch for the per-tensor amax).
 * No reference counterpart beyond the plain cast of utils/fp8_linear.py:12-17; the quantisation rule is
 * defined by this library and restated by the oracle.
 */
int dsb_pack_quant_weight(const void* W, int64_t ld_w, int src_is_bf16, void* Wq, int64_t ld_q, float* scales, int N,
                          int K, int fmt, int per_channel, float* work, void* stream);

/*
 * Quantised Linear that allocates nothing: out = act((quantise_rows(x) . Wq^T) * row_scale * w_scale + bias),
 * i.e. dsb_quant_rows followed by dsb_gemm, with the 8-bit activation copy and the row scales kept in a
 * fixed __device__ array inside the library instead of caller-provided scratch.  For callers that cannot
 * allocate device memory (a plugin inside another runtime's fixed memory plan, an FFI binding that only passes
 * the tensors it was given).  This entry point has no counterpart in the reference.
 *   x: bf16 [M, ld_x]; Wq: [N, ld_w] in w_fmt (E4M3 or INT8); w_scale: 1 or N floats (w_scale_stride 0 or 1);
 *   bias fp32 [N] or NULL; act = DSB_ACT_*; out: bf16 [M, ld_out].  K must be a multiple of 16.
 * Limits: M*K <= 64 Mi elements and M <= 65536, else DSB_ERR_TOO_LARGE.  The array (64.25 MiB) is resident on
 * every GPU that loads the library.  All calls share it: calls that overlap on the GPU race, so serialise them.
 * The first call on each device looks up the array's device address; make that call outside stream capture.
 */
int dsb_linear_static(const void* x, int64_t ld_x, const void* Wq, int64_t ld_w, int w_fmt, int M, int N, int K,
                      const float* w_scale, int w_scale_stride, const float* bias, int act, void* out,
                      int64_t ld_out, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSB_H_ */
