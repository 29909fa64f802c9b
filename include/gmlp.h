/* gmlp.h — C ABI of libgmlp.so, the sm_100a (B200) gated-MLP kernel library.
 *
 * The library replaces the device side of matteobonotto/triton-gated-mlp's fused
 * gated MLP. Each entry point names the reference interface it stands in for
 * (paths are relative to the reference project's root).
 *
 * Conventions
 *   - M = tokens (rows of x), K = hidden size, N = intermediate size, the letters
 *     the reference uses (README.md:32-34). nn.Linear storage: W_gate, W_up are
 *     [N, K]; W_down is [K, N]; every matrix is row-major with the row pitch
 *     given in elements (a multiple of 8) and a 16-byte aligned base address.
 *   - All pointers are DEVICE pointers owned by the caller. Nothing is allocated
 *     or freed by the library and nothing is retained after a call returns (the
 *     one exception, gmlp_peer_alloc / gmlp_peer_free, is a set-up call and says so).
 *   - `stream` is a cudaStream_t passed as void*. Work is enqueued on it and the
 *     call returns without synchronising. The caller makes the right device
 *     current before calling.
 *   - Return value: 0 on success, a negative gmlp_status_t otherwise; the text of
 *     the last error of the calling thread is available from gmlp_last_error().
 *     The library never throws, aborts or falls back to a CPU path.
 *   - Device-side waits are bounded. A kernel that gives up a wait stores a
 *     non-zero code in a per-device status word that gmlp_status_read() returns.
 */
#ifndef GMLP_H
#define GMLP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum gmlp_status_t {
  GMLP_OK = 0,
  GMLP_ERR_SHAPE = -1,    /* a dimension is <= 0, or K/N not a multiple of 8 */
  GMLP_ERR_ALIGN = -2,    /* base address not 16-byte aligned or pitch not a multiple of 8 */
  GMLP_ERR_DTYPE = -3,    /* dtype is not a gmlp_dtype_t, or not one this entry point takes */
  GMLP_ERR_ARCH = -4,     /* current device is not compute capability 10.x */
  GMLP_ERR_LAUNCH = -5,   /* CUDA reported an error while encoding descriptors or launching */
  GMLP_ERR_ARG = -6,      /* NULL where a pointer is required, bad dropout_p, ... */
  GMLP_ERR_SCRATCH = -7   /* scratch buffer too small */
} gmlp_status_t;

/* GMLP_F32: fp32 matrices whose products are taken in tf32 (tcgen05.mma.kind::tf32, fp32
 * accumulation), for modules kept in fp32 as the reference's own tests build them
 * (tests/test_gated_mlp_fwd.py:23-38). Accepted by gmlp_hidden_fwd(_scaled), gmlp_down_fwd,
 * gmlp_mlp_fwd, gmlp_gemm with both operands K-major (a_mn = b_mn = 0), gmlp_bwd_dact and
 * gmlp_colsum; every other entry point answers GMLP_ERR_DTYPE. A compatibility path: the 16-bit
 * types are the tuned ones. */
typedef enum gmlp_dtype_t { GMLP_BF16 = 0, GMLP_FP16 = 1, GMLP_F32 = 2 } gmlp_dtype_t;

/* Gate activations: the names the reference's module accepts (ACT_FWD,
 * src/triton_gated_mlp/gated_mlp.py:27-37); its fused kernels implement only silu and
 * no_act (ops/act.py:7-12) and its backward only silu (gated_mlp.py:46-55). */
typedef enum gmlp_act_t {
  GMLP_ACT_SILU = 0,       /* also "swish" */
  GMLP_ACT_NONE = 1,       /* "no_act": h = g * u */
  GMLP_ACT_RELU = 2,
  GMLP_ACT_GELU = 3,       /* exact (erf) form, nn.GELU's default */
  GMLP_ACT_SIGMOID = 4,
  GMLP_ACT_TANH = 5,
  GMLP_ACT_LEAKY_RELU = 6  /* negative slope 0.01, nn.LeakyReLU's default */
} gmlp_act_t;

/* One gated-MLP problem (or one rank's shard of it).
 * Dropout uses the Philox4x32-10 contract of oracle/philox.py: the keep bit of
 * hidden element (row, col) depends only on (seed, offset) and on its GLOBAL
 * index (row0_global + row) * N_global + (col0_global + col), so token-sharded
 * and intermediate-sharded ranks reproduce the single-GPU mask. */
typedef struct gmlp_problem_t {
  int64_t M;            /* local token rows */
  int64_t K;            /* hidden size */
  int64_t N;            /* local intermediate columns */
  int32_t dtype;        /* gmlp_dtype_t of every matrix and bias vector */
  float dropout_p;      /* 0 disables dropout; must be in [0, 1) */
  uint64_t seed;        /* Philox key */
  uint64_t offset;      /* Philox counter words 2..3; advance once per module call */
  int64_t row0_global;  /* global index of local row 0 (token sharding) */
  int64_t col0_global;  /* global index of local intermediate column 0 (TP sharding) */
  int64_t N_global;     /* un-sharded intermediate size; 0 means N */
  int32_t act;          /* gmlp_act_t of the gate (0 = SiLU) */
  uint32_t tuning;      /* per-call GEMM tuning, GMLP_TUNE_* fields ORed together; 0 = the defaults */
} gmlp_problem_t;

/* Fields of gmlp_problem_t.tuning. A field left 0 takes the process-wide default
 * (the built-in rule unless a gmlp_set_* call changed it). Because the values travel
 * with the call, two modules, host threads or devices never change each other's grids.
 * No counterpart in the reference, which fixes these through its autotuner
 * (src/triton_gated_mlp/ops/fwd.py:48-62). */
#define GMLP_TUNE_PAIR_MODE(m) ((uint32_t)(m) & 3u)               /* 1 single-CTA kernel, 2 CTA pair */
#define GMLP_TUNE_RASTER_GROUP(g) (((uint32_t)(g) & 0xFFFu) << 2)  /* row tiles per raster group */
#define GMLP_TUNE_SM_LIMIT(n) (((uint32_t)(n) & 0xFFFu) << 14)     /* SMs a GEMM grid may occupy */
/* gmlp_decode_fwd*: launch the first kernel as an ordinary kernel instead of a programmatic
 * dependent, so that it reads no weight before everything ahead of it on the stream has
 * finished. For the call that follows a kernel which WRITES the weights (optimiser step,
 * dequantisation, weight merge). */
#define GMLP_TUNE_ORDINARY_LAUNCH (1u << 26)
/* Plain-store GEMMs (down projection, dx, weight gradients) may run on 256 x 512 tiles per CTA pair (one
 * accumulator buffer, a quarter fewer operand bytes per flop) when that shortens the schedule; this bit keeps
 * the call on 256 x 256 tiles. The result is the same bit for bit either way. */
#define GMLP_TUNE_NARROW_TILES (1u << 27)

/* H[M,N] = dropout(act(x W_gate^T + b_gate) * (x W_up^T + b_up)), act = p->act (SiLU by default).
 * Replaces mlp_hidden_states_fwd (src/triton_gated_mlp/ops/fwd.py:198-279, kernel
 * :65-166) with the bias and dropout that EagerGatedMLP applies
 * (src/triton_gated_mlp/gated_mlp.py:96). b_gate / b_up may be NULL.
 * g_save / u_save: both NULL, or both [M,N] buffers that receive the biased
 * pre-activations for the backward pass. */
int gmlp_hidden_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate,
                    const void* b_gate, const void* w_up, const void* b_up, void* h,
                    void* g_save, void* u_save, void* stream);

/* ---- RMSNorm ahead of the MLP (no counterpart in the reference, whose module starts at
 * the projections, src/triton_gated_mlp/gated_mlp.py:224-227; this is the step that
 * precedes it in a Llama block: y = MLP(x / rms(x) * weight)) ----
 * gmlp_rms_rowscale: rs[m] = 1 / sqrt(mean_k x[m,k]^2 + eps) as fp32 [M]; when xn is not
 * NULL also xn[m,k] = x[m,k] * rs[m] ([M,K], contiguous, x's type). x has row pitch ld.
 * gmlp_hidden_fwd_scaled: gmlp_hidden_fwd with both accumulators multiplied by
 * row_scale[row] (fp32 [M], may be NULL) before the bias is added. With
 * W' = W * diag(norm weight) folded on the host this gives
 * act((x / rms * weight) W_gate^T + b_gate) * (... W_up^T + b_up) without the normalised
 * activations ever being written.
 * gmlp_rms_bwd: the backward of xn = x * rs:
 * dx[m,:] = rs[m] * (dxn[m,:] - xn[m,:] * mean_k(dxn[m,k] * xn[m,k])). */
int gmlp_rms_rowscale(int64_t M, int64_t K, int32_t dtype, const void* x, int64_t ld, float eps,
                      float* rs, void* xn, void* stream);
int gmlp_hidden_fwd_scaled(const gmlp_problem_t* p, const void* x, const float* row_scale,
                           const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                           void* h, void* g_save, void* u_save, void* stream);
int gmlp_rms_bwd(int64_t M, int64_t K, int32_t dtype, const void* dxn, const void* xn, const float* rs,
                 void* dx, void* stream);

/* y[M,K] = h W_down^T (+ b_down) (+ residual[M,K]).
 * Replaces self.down_proj(hidden_states) (src/triton_gated_mlp/gated_mlp.py:236). */
int gmlp_down_fwd(const gmlp_problem_t* p, const void* h, const void* w_down,
                  const void* b_down, const void* residual, void* y, void* stream);

/* dH = dy W_down, then d_gate = dH' * u * silu'(g), d_up = dH' * silu(g) with
 * dH' = dH * mask / (1-p), in one kernel. Replaces the dH half of down_proj's
 * autograd (implicit at src/triton_gated_mlp/gated_mlp.py:236) fused with
 * _compute_quantities_for_bwd (src/triton_gated_mlp/ops/bwd.py:82-211), reading
 * the saved pre-activations instead of recomputing them. d_gate may be g and d_up may
 * be u (in place: every element is read before the same thread overwrites it). */
int gmlp_bwd_dhidden(const gmlp_problem_t* p, const void* dy, const void* w_down,
                     const void* g, const void* u, void* d_gate, void* d_up, void* stream);

/* The whole forward pass in one call: gmlp_hidden_fwd then gmlp_down_fwd on `stream`
 * (FusedGatedMLP.forward, src/triton_gated_mlp/gated_mlp.py:222-237: the fused hidden
 * state followed by self.down_proj). Arguments as for the two calls. */
int gmlp_mlp_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate, const void* b_gate,
                 const void* w_up, const void* b_up, const void* w_down, const void* b_down,
                 const void* residual, void* h, void* g_save, void* u_save, void* y, void* stream);

/* The whole backward pass in one call (FusedGatedMLPFunction.backward,
 * src/triton_gated_mlp/gated_mlp.py:186-200, plus the down projection's and the biases'
 * gradients that the reference leaves to autograd): gmlp_bwd_dhidden, gmlp_bwd_dx,
 * gmlp_bwd_dw_gate_up_bias, gmlp_bwd_dw_down_bias, in that order on `stream`.
 * Output pointers that are NULL are skipped: dx; dw_gate and dw_up (both or neither);
 * dw_down; db_gate / db_up (only together with dw_gate, dw_up) and db_down (only with
 * dw_down). d_gate / d_up are work buffers [M,N], required when dx or dw_gate is asked
 * for; they may be the buffers g / u themselves (every element is read before it is
 * overwritten). `scratch` as for gmlp_bwd_dw_gate_up_bias; may be NULL when no bias
 * gradient is asked for. */
int gmlp_mlp_bwd(const gmlp_problem_t* p, const void* dy, const void* x, const void* w_gate,
                 const void* w_up, const void* w_down, const void* g, const void* u, const void* h,
                 void* d_gate, void* d_up, void* dx, void* dw_gate, void* dw_up, void* dw_down,
                 void* db_gate, void* db_up, void* db_down, void* scratch, size_t scratch_bytes,
                 void* stream);

/* The elementwise half of the above for a caller that already holds dH[M,N]
 * (the op-level contract of mlp_hidden_states_bwd, ops/bwd.py:466-602). */
int gmlp_bwd_dact(const gmlp_problem_t* p, const void* dh, const void* g, const void* u,
                  void* d_gate, void* d_up, void* stream);

/* dx[M,K] = d_gate W_gate + d_up W_up. Replaces _compute_dx (ops/bwd.py:231-322). */
int gmlp_bwd_dx(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                const void* w_gate, const void* w_up, void* dx, void* stream);

/* dW_gate[N,K] = d_gate^T x, dW_up[N,K] = d_up^T x (full reduction over all M
 * rows). Replaces _compute_dW_up_dW_gp (ops/bwd.py:379-463). */
int gmlp_bwd_dw_gate_up(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                        const void* x, void* dw_gate, void* dw_up, void* stream);

/* dW_down[K,N] = dy^T h. Replaces the weight-gradient half of down_proj's
 * autograd (implicit at src/triton_gated_mlp/gated_mlp.py:236). */
int gmlp_bwd_dw_down(const gmlp_problem_t* p, const void* dy, const void* h, void* dw_down,
                     void* stream);

/* The two weight-gradient GEMMs above with the bias gradients fused in:
 * db_gate[N] = sum over tokens of d_gate, db_up[N] likewise, db_down[K] = sum over
 * tokens of dy. The reference returns None for the gate / up bias gradients
 * (src/triton_gated_mlp/gated_mlp.py:200) and leaves db_down to autograd of :236;
 * EagerGatedMLP's autograd defines the values. The sums are the row sums of the GEMM's
 * own A operand (d^T), taken beside the main loop by an otherwise idle warp of every
 * CTA from tiles fetched a second time through L2: no extra launch and no second pass
 * over d_gate / d_up / dy in HBM. Any of the db pointers may be NULL (with all NULL
 * the call is the plain GEMM and takes no scratch). fp32 accumulation, partial sums
 * added in a fixed order: results are bitwise repeatable.
 * `scratch`: gmlp_bias_grad_scratch_bytes(p) bytes, 16-byte aligned, serves both calls;
 * its first 64 KiB (arrival counters) must be ZERO before the first call and every
 * call leaves them zero, unless gmlp_status_read has since returned a non-zero word:
 * then clear them again. Calls that share a scratch buffer must not overlap on the GPU. */
size_t gmlp_bias_grad_scratch_bytes(const gmlp_problem_t* p);
int gmlp_bwd_dw_gate_up_bias(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                             const void* x, void* dw_gate, void* dw_up, void* db_gate, void* db_up,
                             void* scratch, size_t scratch_bytes, void* stream);
int gmlp_bwd_dw_down_bias(const gmlp_problem_t* p, const void* dy, const void* h, void* dw_down,
                          void* db_down, void* scratch, size_t scratch_bytes, void* stream);

/* dst[cols] = sum over rows of src[rows, cols] (fp32 accumulation): the bias
 * gradients db_gate, db_up (from d_gate, d_up) and db_down (from dy), which the
 * reference leaves to autograd of nn.Linear / returns as None
 * (src/triton_gated_mlp/gated_mlp.py:200), as a stand-alone pass for a caller that
 * does not run the weight-gradient GEMMs (which otherwise deliver them, see above).
 * `scratch` holds gmlp_colsum_scratch_bytes(rows, cols) bytes of fp32 partial sums. */
size_t gmlp_colsum_scratch_bytes(int64_t rows, int64_t cols);
int gmlp_colsum(int64_t rows, int64_t cols, int32_t dtype, const void* src, int64_t ld,
                void* scratch, size_t scratch_bytes, void* dst, void* stream);

/* gmlp_colsum for callers that cannot hand over scratch memory. It has no counterpart
 * in the reference. Same result as gmlp_colsum, but the fp32 partial sums go to a 1 MiB
 * array inside the library image (every GPU that loads the library holds that 1 MiB
 * until the process exits), and the call makes no cudaMalloc / cudaFree or any other
 * allocating call. It is meant for hosts that bind this ABI from a runtime which gave
 * all device memory to its own pool at start-up (so there is nothing left to allocate
 * from and no torch allocator to ask), or which must not trigger the device-wide
 * synchronisation an allocation implies in the middle of a latency-critical loop.
 *   - Limit: gmlp_colsum_scratch_bytes(rows, cols) <= 1 MiB, which holds for every
 *     cols <= 262144 at any row count. Wider matrices are refused with
 *     GMLP_ERR_SCRATCH and a message; use gmlp_colsum for them.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call before
 *     starting any stream capture. The first libgmlp call of any kind on a device is
 *     also when the CUDA runtime loads the library's device image, this array
 *     included: a host that is about to hand all remaining device memory to its own
 *     pool must make one libgmlp call on every device BEFORE it does so, or the image
 *     finds no room.
 *   - All calls on a device share the one array. It keeps whatever the last call left
 *     there, which is harmless (the first pass overwrites every value the second pass
 *     reads), but two calls that overlap on the GPU (different streams) race on it:
 *     serialise them. */
int gmlp_colsum_static(int64_t rows, int64_t cols, int32_t dtype, const void* src, int64_t ld,
                       void* dst, void* stream);

/* Skinny-M (decode) forward for M <= 64 tokens, K and N multiples of 64:
 * h[M,N] = act(x W_gate^T + b_gate) * (x W_up^T + b_up), then y[M,K] = h W_down^T +
 * b_down (+ residual[M,K], may be NULL), as two weight-streaming kernels (HBM-bound; every weight byte is read
 * once). Covers the same reference interfaces as gmlp_hidden_fwd + gmlp_down_fwd
 * (src/triton_gated_mlp/ops/fwd.py:198-279 and gated_mlp.py:236) for the token
 * counts at which the reference's smallest tile (BLOCK_SIZE_M = 16, ops/fwd.py:49)
 * already wastes the tensor pipe. dropout_p must be 0.
 * `scratch`: gmlp_decode_scratch_bytes(p) bytes, 16-byte aligned. Its leading
 * counter area (the first 64 KiB is more than enough) must be ZERO before the first
 * call; every call leaves it zero again, so one memset at allocation suffices, with
 * one exception: after gmlp_status_read has returned a non-zero word (a kernel gave
 * up a wait) the counter area must be cleared again before the scratch is reused.
 * Calls that share a scratch buffer must not overlap on the GPU.
 * Both kernels start as programmatic dependents of whatever precedes them on
 * `stream` and begin streaming WEIGHTS before that predecessor has finished (they
 * wait for it only before touching x, h, y or the scratch). The kernel immediately
 * before the call on the stream must therefore not write w_gate, w_up or w_down:
 * after an optimiser step, a dequantisation or a weight merge into those buffers,
 * set GMLP_TUNE_ORDINARY_LAUNCH in p->tuning for that call (or put any other kernel
 * or an event wait between the writer and the call). */
size_t gmlp_decode_scratch_bytes(const gmlp_problem_t* p);
int gmlp_decode_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate,
                    const void* b_gate, const void* w_up, const void* b_up, const void* w_down,
                    const void* b_down, const void* residual, void* h, void* y, void* scratch,
                    size_t scratch_bytes, void* stream);

/* gmlp_decode_fwd with the gate / up accumulators multiplied by row_scale[token] (fp32 [M],
 * may be NULL) before the bias: the RMSNorm prologue of gmlp_hidden_fwd_scaled on the decode path. */
int gmlp_decode_fwd_scaled(const gmlp_problem_t* p, const void* x, const float* row_scale,
                           const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                           const void* w_down, const void* b_down, const void* residual, void* h, void* y,
                           void* scratch, size_t scratch_bytes, void* stream);

/* gmlp_decode_fwd_scaled from ONE kernel launch (bf16 / fp16): a persistent kernel streams W_gate and
 * W_up, then runs on into W_down without draining its operand ring; the CTAs hand the columns of H
 * to each other through a device-wide count in the scratch instead of a kernel boundary. Same
 * arguments, scratch (gmlp_decode_scratch_bytes), preconditions and result as the two-launch form.
 * All CTAs of the grid (one per SM) must be able to run at the same time: launched beside another
 * kernel that holds SMs for about a second, its waits run out and the status word is set. Replaces the
 * reference's two separate steps src/triton_gated_mlp/gated_mlp.py:227-236 for small batches. */
int gmlp_decode_fwd_fused(const gmlp_problem_t* p, const void* x, const float* row_scale,
                          const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                          const void* w_down, const void* b_down, const void* residual, void* h, void* y,
                          void* scratch, size_t scratch_bytes, void* stream);

/* ---- decode with 8-bit (e4m3) weights: half the bytes of the HBM-bound weight stream ----
 * No counterpart in the reference (its benchmark runs fp16 only,
 * src/triton_gated_mlp/benchmark.py:26-123). Weights are e4m3 bytes with one fp32 scale per
 * weight ROW (W ~= w8 * scale[row]; prepared once by the host); activations are quantised
 * per TOKEN on the fly by gmlp_quantize_rows_e4m3; both operands go to
 * tcgen05.mma.kind::f8f6f4 (fp32 accumulation) and the accumulators are multiplied by
 * (token scale * weight-row scale) before bias and activation.
 * gmlp_quantize_rows_e4m3: scale[m] = max(amax_k |x[m,k]|, 1e-30) / 448;
 *   q[m,k] = e4m3(x[m,k] / scale[m]) (round to nearest even, saturating). q is [M,K] bytes.
 * gmlp_decode_fwd_fp8: x [M,K] 16-bit in; work buffers x8 [M,K] bytes, x_scale [M],
 *   h [M,N] 16-bit, h8 [M,N] bytes, h_scale [M]; y [M,K] 16-bit out. K and N multiples of
 *   128, M <= 64; scratch and the rules about it, about the stream and about what may
 *   precede the call as for gmlp_decode_fwd. Four launches: quantise x, gate/up, quantise
 *   h, down. */
int gmlp_quantize_rows_e4m3(int64_t M, int64_t K, int32_t dtype, const void* x, int64_t ld, void* q,
                            float* scale, void* stream);
int gmlp_decode_fwd_fp8(const gmlp_problem_t* p, const void* x, const void* w_gate8,
                        const float* w_gate_scale, const void* b_gate, const void* w_up8,
                        const float* w_up_scale, const void* b_up, const void* w_down8,
                        const float* w_down_scale, const void* b_down, const void* residual, void* x8,
                        float* x_scale, void* h, void* h8, float* h_scale, void* y, void* scratch,
                        size_t scratch_bytes, void* stream);

/* mask[M,N] (one byte per element, 1 = kept) for the problem's dropout settings:
 * the device side of the bit-exact mask check. */
int gmlp_dropout_mask(const gmlp_problem_t* p, uint8_t* mask, void* stream);

/* C[M,N] = A B^T (+ bias[N]) with fp32 accumulation: the GEMM engine under every
 * call above, exported for its own parity tests. a_mn = 0: A stored [M,K]
 * (K-major); a_mn = 1: A stored [K,M]. b_mn = 0: B stored [N,K]; b_mn = 1: B
 * stored [K,N]. lda / ldb / ldc are row pitches in elements. */
int gmlp_gemm(int32_t dtype, int32_t a_mn, int32_t b_mn, int64_t M, int64_t N, int64_t K,
              const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
              const void* bias, void* stream);

/* Tuning / test hook with no counterpart in the reference: which GEMM kernel the
 * calls above launch. 0 (default) = per problem, 1 = always the single-CTA kernel
 * (128-row tiles), 2 = always the CTA-pair kernel (256-row tiles on two SMs,
 * tcgen05 cta_group::2). Returns the previous mode; other values only query. */
int gmlp_set_cta_pair_mode(int mode);

/* Tuning hook with no counterpart in the reference (the reference autotunes its
 * GROUP_SIZE_M, src/triton_gated_mlp/ops/fwd.py:48-62): row tiles per raster
 * group of the persistent tile order; 0 restores the built-in default. Returns
 * the previous value; values outside [0, 4096] only query. */
int gmlp_set_raster_group(int row_tiles);

/* Scheduling hook with no counterpart in the reference: the number of SMs the
 * persistent GEMM grids of the calls above may occupy (0 = all, the default). A host
 * that overlaps a collective (NCCL) with the GEMMs lowers it for those launches so
 * that the collective's CTAs find free SMs; with every SM held by a persistent CTA
 * they would wait for the GEMM to end. Returns the previous value; values outside
 * [0, 4096] only query. Decode and elementwise kernels are not affected. */
int gmlp_set_sm_limit(int sms);

/* ---- tensor-parallel output sum over peer memory (no reference counterpart: the
 * reference is single-GPU; this replaces an NCCL all-reduce after gmlp_down_fwd /
 * gmlp_decode_fwd when the intermediate dimension is sharded) ----
 *
 * Each rank owns one REGION of gmlp_peer_region_bytes(max_elems, world) bytes that
 * every other rank of the group has mapped: inbox slots the peers push their
 * partials into, flag words and the rank's own call counters (layout in
 * csrc/peer_reduce.cuh). gmlp_peer_alloc is a control-plane call, once per group:
 * it cudaMalloc's `bytes` of zeroed device memory on the current device and exports
 * it as 64 opaque bytes (a CUDA IPC handle) that the other ranks' processes pass to
 * gmlp_peer_open to map it (peer access over NVLink is enabled on first use).
 * gmlp_peer_close unmaps, gmlp_peer_free releases. The hosts exchange the handles
 * themselves (torch.distributed.all_gather_object in the Python layer) and must
 * not start reducing before every rank has allocated and mapped.
 *
 * gmlp_peer_allreduce: dst[i] = sum over ranks of src[i] (fp32 accumulation in rank
 * order, so every rank gets the same bits) for n <= max_elems elements (a multiple
 * of 8) of `dtype`; dst may be src. `regions` is a HOST array of `world` device
 * pointers, regions[p] = rank p's region (local for p == rank, else as mapped by
 * gmlp_peer_open); max_elems is the capacity the regions were sized with. Every
 * rank of the group must make the same sequence of calls (same n). The call number
 * is kept on the device, so a call carries no per-call host state. src must be
 * complete on `stream` before the call. `dependent` != 0 launches the kernel as a
 * programmatic dependent of the preceding kernel on the stream (which must be the
 * one that wrote src). One kernel, no allocation, no host synchronisation: every
 * partial is pushed to every peer, except from 1 MB on with eight ranks (and n a
 * multiple of 8 * world), where each rank reduces one slice and hands the result
 * round. The wait for the peers is bounded (about a second); on expiry dst is left
 * unwritten and gmlp_status_read returns 4. Calls that share regions must not overlap on a
 * GPU (one stream per group). */
/* Tuning / test hook: the size in bytes from which gmlp_peer_allreduce takes the
 * two-shot form. 0 = the built-in rule below, > 0 = from that many bytes at any group
 * size, < 0 = never. Every rank must use the same setting. Returns the previous one. */
long long gmlp_set_peer_two_shot_bytes(long long bytes);
size_t gmlp_peer_region_bytes(int64_t max_elems, int32_t world);
int gmlp_peer_alloc(size_t bytes, void** ptr, void* handle64);
int gmlp_peer_open(const void* handle64, void** ptr);
int gmlp_peer_close(void* ptr);
int gmlp_peer_free(void* ptr);
int gmlp_peer_allreduce(int32_t dtype, int64_t n, int64_t max_elems, const void* src,
                        void* const* regions, int32_t rank, int32_t world, void* dst,
                        int32_t dependent, void* stream);

/* ---- tensor-parallel down projection that scatters while it computes ----
 * gmlp_down_fwd_push is gmlp_down_fwd (the step src/triton_gated_mlp/gated_mlp.py:236 of the reference,
 * on this rank's shard of the intermediate dimension) whose epilogue sends every finished block
 * of the partial y to the rank that owns its rows: rank r owns rows [r M / world, (r + 1) M / world);
 * blocks of this rank's own rows are stored to y as usual, all others go with plain peer stores over
 * NVLink into the owner's inbox (regions / max_elems as for gmlp_peer_allreduce, sized for
 * M * K elements) while the remaining tiles are still being computed: the scatter half of a
 * reduce-scatter inside the GEMM. gmlp_peer_reduce_gather, enqueued behind it on the same stream by
 * every rank, raises and awaits the flags, adds the world partials of this rank's rows in rank order in
 * fp32, writes them to y and hands them round, so that y ends as the full sum on every rank (identical
 * bits). M must be a multiple of 32 * world, n = M * K a multiple of 8 * world; y contiguous. The
 * two calls form one step of the call sequence all ranks share; regions used this way must not be
 * used by plain gmlp_peer_allreduce calls in between on another stream. Waits are bounded as there. */
int gmlp_down_fwd_push(const gmlp_problem_t* p, const void* h, const void* w_down, const void* b_down,
                       const void* residual, void* y, int64_t max_elems, void* const* regions, int32_t rank,
                       int32_t world, void* stream);
int gmlp_peer_reduce_gather(int32_t dtype, int64_t n, int64_t max_elems, void* y, void* const* regions,
                            int32_t rank, int32_t world, void* stream);
/* The same scatter from the epilogue of gmlp_bwd_dx (dx is the other tensor-parallel partial sum, over the
 * shards of the intermediate dimension; _compute_dx in src/triton_gated_mlp/ops/bwd.py:231-322). The
 * gmlp_peer_reduce_gather(dx) that completes it may be enqueued later on the stream, e.g. behind the
 * weight-gradient GEMMs, as long as no other call uses the regions in between. */
int gmlp_bwd_dx_push(const gmlp_problem_t* p, const void* d_gate, const void* d_up, const void* w_gate,
                     const void* w_up, void* dx, int64_t max_elems, void* const* regions, int32_t rank,
                     int32_t world, void* stream);

/* Reads and clears the current device's status word (synchronises the device).
 * 0 = no kernel gave up a wait since the last read. */
int gmlp_status_read(int* value);

const char* gmlp_last_error(void);
int gmlp_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GMLP_H */
