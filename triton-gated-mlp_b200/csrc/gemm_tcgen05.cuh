// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused gated-MLP
// epilogues. One CTA per SM walks a grouped tile order; per CTA:
//   warp 0 (one lane)  TMA producer: fills a STAGES-deep shared-memory ring
//   warp 1 (one lane)  MMA issuer: tcgen05.mma into one of two TMEM accumulators
//   warps 2..17        epilogue: tcgen05.ld the finished accumulator, apply the
//                      fused elementwise work, hand the result to TMA stores
//   warp 18            watcher: waits for "accumulator full" and wakes the epilogue
//                      warps, which sleep at a named barrier meanwhile
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of
// tile i+1. No TMA multicast is used.
//
// Logical problem: C[M, N] = sum_k A[m, k] * B[n, k], 16-bit inputs, fp32
// accumulation. Each operand can be stored K-major (reduction index contiguous)
// or MN-major (m or n contiguous, one row per reduction index), which covers
// every product of the gated-MLP forward and backward without a transpose pass.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "philox.cuh"
#include "sm100_ptx.cuh"

namespace gmlp {

enum : int {
  EPI_STORE = 0,    // C (+ bias[n]) (+ residual[m, n])            -> out0 / out1 (per batch)
  EPI_SWIGLU = 1,   // accumulator = [gate | up] per tile; H = dropout(silu(g) * u)
  EPI_DHIDDEN = 2,  // accumulator = dH; reads G, U; writes dGate, dUp
};

enum : int {
  GMLP_DEV_TIMEOUT_PRODUCER = 1,
  GMLP_DEV_TIMEOUT_MMA = 2,
  GMLP_DEV_TIMEOUT_EPILOGUE = 3,
};

struct GemmArgs {
  int M;        // output rows
  int N;        // output columns (EPI_SWIGLU: hidden columns; the accumulator holds 2 per column)
  int kb0;      // 64-element reduction blocks taken from (A0, B0)
  int kb1;      // 64-element reduction blocks taken from (A1, B1) afterwards (0 = unused)
  int batches;  // 1, or 2: two problems (A0 -> out0, A1 -> out1) that share B0
  int group_m;  // row tiles per raster group
  int act;      // gate activation (ACT_*)
  uint32_t idesc;
  int* status;  // device word; a role that gives up a wait stores its code here
  void* out0;
  void* out1;
  void* out2;
  const void* in0;
  const void* in1;
  const void* bias0;
  const void* bias1;
  const float* row_scale;  // EPI_SWIGLU: optional [M] factors applied to both accumulators before the bias
                           // (1 / rms of the input row when an RMSNorm precedes the MLP)
  long long ld_out;  // row pitch (elements) of out*
  long long ld_in;   // row pitch (elements) of in*
  DropoutParams drop;
  // Row sums of an MN-major A operand, taken on the side by the watcher warp (ASUM kernels):
  // the bias gradients of the weight-gradient GEMMs, db[n] = sum over tokens of d[token, n],
  // where d^T is exactly the kernel's A. Null / zero when unused.
  void* asum_out[2];  // per batch: [M] sums, in the matrices' 16-bit type
  float* asum_part;   // [batches][n_tiles][m_tiles * tile rows] fp32 partial sums
  int* asum_cnt;      // [batches][m_tiles * tile rows / 128] arrivals; zero on entry and on exit
  // Tensor-parallel down projection (EPI_STORE): the row blocks of the output belong to the ranks in
  // contiguous shares of push_rows rows. A finished block of a row that another rank owns does not go to
  // out0 but straight into that rank's inbox (plain peer stores over NVLink), at the same [row, column]
  // offset: the scatter half of a reduce-scatter, done tile by tile from the GEMM's epilogue while the other
  // tiles are still being computed. push_world = 0: off.
  char* push_base[8];          // per rank: its inbox slot for this rank's partials, parity 0
  long long push_parity_bytes; // distance to the same slot of parity 1
  const unsigned int* push_epoch;  // calls completed by this rank's sum kernel: the next call's number is +1
  int push_rows;               // rows per owner (a multiple of 32)
  int push_rank, push_world;
};

constexpr int BM = 128;        // rows per tile = TMEM lanes
constexpr int BK = 64;         // reduction elements per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;     // reduction elements per tcgen05.mma (16-bit inputs)

// Epilogue warps, and who wakes them. The sixteen epilogue warps have nothing to do for
// most of a tile's main loop. Polling the "accumulator full" mbarrier from each of them
// issues instructions the whole time, which on a power-capped part costs clock; so they
// sleep at a named barrier (no issue slots) and ONE watcher warp polls the mbarrier and
// arrives on the named barrier for them. The watcher also decides, once per tile and
// for all epilogue warps alike, whether the tile is processed or the kernel is being
// abandoned (epi_go), so the warps can never take different ways out.
constexpr int EPI_WARPS = 16;
constexpr int WATCHER_WARP = 2 + EPI_WARPS;
constexpr int GEMM_THREADS = 32 * (3 + EPI_WARPS);        // 608
constexpr uint32_t EPI_BAR_THREADS = 32 * (EPI_WARPS + 1);  // epilogue warps + watcher
constexpr uint32_t EPI_BAR_ID0 = 1;                       // named barriers 1, 2: one per accumulator
#ifndef GMLP_PRODUCER_SLEEP_NS
#define GMLP_PRODUCER_SLEEP_NS 100
#endif
#ifndef GMLP_WATCHER_SLEEP_NS
#define GMLP_WATCHER_SLEEP_NS 400
#endif
constexpr int PRODUCER_SLEEP_NS = GMLP_PRODUCER_SLEEP_NS;  // between polls of a full ring (stages ahead of the MMAs)
constexpr int WATCHER_SLEEP_NS = GMLP_WATCHER_SLEEP_NS;    // between polls for a tile's completion (10 us or more apart)
constexpr uint32_t EPI_DONE_BAR = 3;                      // ASUM kernels: the epilogue warps have left the staging area
constexpr int ASUM_BUFS = 4;                              // the watcher's private ring: 4 x 16 KB in the staging area

__host__ __device__ constexpr uint32_t tmem_cols_for(int bn) {
  return (2 * bn <= 32) ? 32u : (2 * bn <= 64) ? 64u : (2 * bn <= 128) ? 128u
         : (2 * bn <= 256) ? 256u : 512u;
}

// Epilogue staging (see "Epilogue I/O" below).
constexpr int EPI_PARTS = EPI_WARPS / 4;  // column parts of a tile
constexpr int BLK_BYTES = 32 * 32;        // dH epilogue: one warp's [32 rows x 16 columns] 16-bit block
constexpr int STORE_STAGE_BYTES = 4096;   // every epilogue: 4 KB of staging per warp
template <int EPI>
__host__ __device__ constexpr int staging_bytes() {
  return EPI_WARPS * STORE_STAGE_BYTES;
}
// Ring depth: as many stages as fit beside the staging area in the 227 KB a CTA may use.
constexpr int SMEM_LIMIT = 232448;
template <int B_ROWS, int EPI>
__host__ __device__ constexpr int gemm_stages() {
  return (SMEM_LIMIT - 2048 - staging_bytes<EPI>()) / (BM * 128 + B_ROWS * 128);
}
// Operand ring (B_ROWS rows of B per stage and CTA) + staging + alignment slack.
template <int B_ROWS, int EPI, int STAGES>
constexpr size_t gemm_smem_bytes() {
  return static_cast<size_t>(STAGES) * (BM * 128 + B_ROWS * 128) + staging_bytes<EPI>() + 1024;
}

// ------------------------------------------------------------ small helpers --
template <typename T>
struct Pack2;
template <>
struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  }
};
template <>
struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = Pack2<T>::unpack(q.x), b = Pack2<T>::unpack(q.y), c = Pack2<T>::unpack(q.z),
         d = Pack2<T>::unpack(q.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
  uint4 q;
  q.x = Pack2<T>::pack(v[0], v[1]);
  q.y = Pack2<T>::pack(v[2], v[3]);
  q.z = Pack2<T>::pack(v[4], v[5]);
  q.w = Pack2<T>::pack(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

// fp32 matrices (the tf32 path): eight consecutive values are two 16-byte accesses.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
// Reduction elements in one 128-byte row of an operand tile: 64 for the 16-bit types, 32 for fp32.
template <typename T>
__host__ __device__ constexpr int row_elems() {
  return 128 / static_cast<int>(sizeof(T));
}

// sigma(x) = 1 / (1 + e^-x) = 0.5 * tanh(x / 2) + 0.5: one MUFU op and two FMAs. The
// hardware tanh approximation has a maximum relative error of about 2^-11, far below
// the resolution of the 16-bit outputs.
__device__ __forceinline__ float sigmoid_f(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
}

// Gate activations (the names the reference's module accepts, gated_mlp.py:17-37).
enum : int {
  ACT_SILU = 0,
  ACT_NONE = 1,
  ACT_RELU = 2,
  ACT_GELU = 3,  // exact (erf) form, nn.GELU's default
  ACT_SIGMOID = 4,
  ACT_TANH = 5,
  ACT_LEAKY_RELU = 6,  // negative slope 0.01, nn.LeakyReLU's default
};
__device__ __forceinline__ float tanh_f(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
// f(x) and f'(x) of the gate activation. `act` is uniform over the launch, so the switch
// never diverges.
__device__ __forceinline__ void act_value_grad(int act, float x, float& f, float& df) {
  switch (act) {
    case ACT_SILU: {
      const float s = sigmoid_f(x);
      f = x * s;
      df = s * (1.0f + x * (1.0f - s));
      break;
    }
    case ACT_RELU:
      f = fmaxf(x, 0.0f);
      df = x > 0.0f ? 1.0f : 0.0f;
      break;
    case ACT_GELU: {
      const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
      f = x * cdf;
      df = cdf + x * 0.39894228040143268f * __expf(-0.5f * x * x);
      break;
    }
    case ACT_SIGMOID: {
      const float s = sigmoid_f(x);
      f = s;
      df = s * (1.0f - s);
      break;
    }
    case ACT_TANH: {
      const float t = tanh_f(x);
      f = t;
      df = 1.0f - t * t;
      break;
    }
    case ACT_LEAKY_RELU:
      f = x > 0.0f ? x : 0.01f * x;
      df = x > 0.0f ? 1.0f : 0.01f;
      break;
    default:  // ACT_NONE
      f = x;
      df = 1.0f;
      break;
  }
}
__device__ __forceinline__ float act_value(int act, float x) {
  switch (act) {
    case ACT_SILU: return x * sigmoid_f(x);
    case ACT_RELU: return fmaxf(x, 0.0f);
    case ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case ACT_SIGMOID: return sigmoid_f(x);
    case ACT_TANH: return tanh_f(x);
    case ACT_LEAKY_RELU: return x > 0.0f ? x : 0.01f * x;
    default: return x;
  }
}

// keep/scale factors for the 8 consecutive columns starting at (grow, gcol), gcol a
// multiple of 8 in the global index space: one Philox call, sixteen bits per element.
__device__ __forceinline__ void dropout_factors8(const DropoutParams& d, long long grow,
                                                 long long gcol, float (&f)[8]) {
  const unsigned long long e =
      static_cast<unsigned long long>(grow) * static_cast<unsigned long long>(d.ncols_global) +
      static_cast<unsigned long long>(gcol);
  const Philox4 r = dropout_words(d, e >> 3);
  f[0] = (r.x & 0xFFFFu) >= d.thresh ? d.scale : 0.0f;
  f[1] = (r.x >> 16) >= d.thresh ? d.scale : 0.0f;
  f[2] = (r.y & 0xFFFFu) >= d.thresh ? d.scale : 0.0f;
  f[3] = (r.y >> 16) >= d.thresh ? d.scale : 0.0f;
  f[4] = (r.z & 0xFFFFu) >= d.thresh ? d.scale : 0.0f;
  f[5] = (r.z >> 16) >= d.thresh ? d.scale : 0.0f;
  f[6] = (r.w & 0xFFFFu) >= d.thresh ? d.scale : 0.0f;
  f[7] = (r.w >> 16) >= d.thresh ? d.scale : 0.0f;
}

struct TileCoord {
  int batch, m_tile, n_tile;
};
// Grouped raster: `group_m` row tiles sweep all column tiles before the next
// group starts, so concurrently running CTAs share A and B tiles in L2.
__device__ __forceinline__ TileCoord decode_tile(int tile, int m_tiles, int n_tiles,
                                                 int group_m) {
  TileCoord c;
  const int per_batch = m_tiles * n_tiles;
  c.batch = tile / per_batch;
  int t = tile - c.batch * per_batch;
  const int per_group = group_m * n_tiles;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsize = min(m_tiles - first_m, group_m);
  t -= g * per_group;
  c.m_tile = first_m + (t % gsize);
  c.n_tile = t / gsize;
  return c;
}

// ------------------------------------------------------------ Epilogue I/O ----
// EPI_WARPS = 16 epilogue warps, four per TMEM lane quarter: warp e (0..15) reads TMEM
// lanes 32 * (e & 3) and column part (e >> 2) of the tile.
//
// After tcgen05.ld a thread owns one output ROW. Moving data between global memory and
// that layout directly makes every 16-byte access of a warp touch 32 different cache
// lines, so every epilogue goes through shared memory.
//
// Store and gate/up epilogues: each warp writes its rows into a staging block laid out
// the way a TMA store expects it (rows of 128 or 64 bytes, swizzled in 16-byte chunks so
// that the 32 row-owning lanes hit 32 different bank groups), and one lane hands the whole
// [32 rows x 64 or 32 columns] block to the TMA engine: one bulk store instead of
// st.shared / ld.shared / st.global round trips on the load/store unit, no address
// arithmetic or bounds predicates per access (the TMA engine clips at the matrix edge).
// Rows of 128 bytes where a warp covers 64 columns; the gate/up epilogue covers 32 hidden
// columns per warp and uses 64-byte rows. (TMA requests are counted per row of a box:
// the shorter the row, the more of the engine's request rate a block costs, which is why
// no epilogue uses 32-byte rows.)
//
// dH epilogue: it also LOADS two [M, N] matrices and keeps to the load/store unit: every
// warp owns two PAIRS of 1 KB staging blocks ([32 rows x 16 columns], 32-byte rows; one block
// for G, one for U) and transposes through them, so that in global memory two neighbouring
// lanes cover one row's 32 bytes. The loads are asynchronous copies (cp.async) straight into
// a pair, issued two 16-column units ahead of use (no registers held meanwhile), so the
// first two units of a tile are fetched while the warp sleeps through the main loop.
//   row view        lane r holds row r:            bytes [32 r, 32 r + 32)
//   coalesced view  lane l, step t in {0, 1}:      row (l >> 1) + 16 t, 16-byte half l & 1
// The two halves of a row swap places in rows 4..7 of every group of 8 (a 32-byte
// swizzle), which keeps both views free of bank conflicts. Every element is read and
// then written by the same lane at the same coordinates, so dGate / dUp may be the very
// buffers G / U were read from.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  float2 a = Pack2<T>::unpack(q.x), b = Pack2<T>::unpack(q.y), c = Pack2<T>::unpack(q.z),
         d = Pack2<T>::unpack(q.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 q;
  q.x = Pack2<T>::pack(v[0], v[1]);
  q.y = Pack2<T>::pack(v[2], v[3]);
  q.z = Pack2<T>::pack(v[4], v[5]);
  q.w = Pack2<T>::pack(v[6], v[7]);
  return q;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 q;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
               : "r"(addr)
               : "memory");
  return q;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& q) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(q.x), "r"(q.y),
               "r"(q.z), "r"(q.w)
               : "memory");
}

// Offset of 16-byte chunk `c` of row `r` in a staging block with rows of ROW_BYTES
// (128 or 64), swizzled the way the TMA engine reads it back: the chunk index is XORed
// with bits [7, 7 + log2(ROW_BYTES / 16)) of the byte address.
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t staged_chunk(int r, int c) {
  static_assert(ROW_BYTES == 128 || ROW_BYTES == 64, "row length of a staging block");
  const int x = ROW_BYTES == 128 ? (r & 7) : ((r >> 1) & 3);
  return static_cast<uint32_t>(r * ROW_BYTES + ((c ^ x) << 4));
}

// SiLU on two values at once: sigma(x) = 0.5 tanh(x / 2) + 0.5 with the multiplies and
// FMAs issued as packed fp32 pairs.
__device__ __forceinline__ f32x2 sigmoid2(f32x2 x) {
  const f32x2 half = f2_pack(0.5f, 0.5f);
  float a, b;
  f2_unpack(f2_mul(x, half), a, b);
  return f2_fma(f2_pack(tanh_f(a), tanh_f(b)), half, half);
}

// keep/scale factors for 8 consecutive columns as in dropout_factors8, with the tests
// done on the raw words: (w >> 16) >= t  <=>  w >= (t << 16), and for the low half the
// same after shifting it up.
__device__ __forceinline__ void dropout_factors8_fast(const DropoutParams& d, long long grow,
                                                      long long gcol, float (&f)[8]) {
  const unsigned long long e =
      static_cast<unsigned long long>(grow) * static_cast<unsigned long long>(d.ncols_global) +
      static_cast<unsigned long long>(gcol);
  const Philox4 r = dropout_words(d, e >> 3);
  const uint32_t t = d.thresh << 16;
  f[0] = (r.x << 16) >= t ? d.scale : 0.0f;
  f[1] = r.x >= t ? d.scale : 0.0f;
  f[2] = (r.y << 16) >= t ? d.scale : 0.0f;
  f[3] = r.y >= t ? d.scale : 0.0f;
  f[4] = (r.z << 16) >= t ? d.scale : 0.0f;
  f[5] = r.z >= t ? d.scale : 0.0f;
  f[6] = (r.w << 16) >= t ? d.scale : 0.0f;
  f[7] = r.w >= t ? d.scale : 0.0f;
}

// Addressing of one warp's dH staging blocks for one lane.
struct BlockView {
  uint32_t row_lo, row_hi;   // row view: offsets of this lane's two 16-byte halves
  uint32_t co[2];            // coalesced view: offset of this lane's 16 bytes in step t
  int crow[2];               // coalesced view: row inside the block in step t
  int chalf;                 // coalesced view: which 8-column half this lane covers

  __device__ __forceinline__ explicit BlockView(int lane) {
    const uint32_t sw = static_cast<uint32_t>((lane >> 2) & 1) << 4;
    row_lo = lane * 32 + sw;
    row_hi = lane * 32 + (16u ^ sw);
    chalf = lane & 1;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      crow[t] = (lane >> 1) + 16 * t;
      const uint32_t csw = static_cast<uint32_t>((crow[t] >> 2) & 1) << 4;
      co[t] = crow[t] * 32 + ((static_cast<uint32_t>(chalf) << 4) ^ csw);
    }
  }
};

// Store this warp's [32 x 16] block whose row `lane` is (lo, hi): rows row0.. of `out`,
// columns col..col+15; rows >= M and 8-column halves at or beyond N are skipped.
// `buf` must not be in use by an earlier call that is not separated from this one by a
// __syncwarp(); alternate between the warp's two blocks.
template <typename T>
__device__ __forceinline__ void store_block(const BlockView& bv, uint32_t buf, T* out, long long ld,
                                            int row0, int col, int M, int N, const uint4& lo,
                                            const uint4& hi) {
  st_shared_v4(buf + bv.row_lo, lo);
  st_shared_v4(buf + bv.row_hi, hi);
  __syncwarp();
  const int c = col + bv.chalf * 8;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const uint4 v = ld_shared_v4(buf + bv.co[t]);
    const int r = row0 + bv.crow[t];
    if (r < M && c < N) *reinterpret_cast<uint4*>(out + static_cast<long long>(r) * ld + c) = v;
  }
}
// First half of a block load: this lane's two 16-byte pieces in the coalesced view
// (zero where the block leaves the matrix). Issued one unit ahead of use. Ordinary
// loads, not the read-only path: the block may be overwritten in place later on.
template <typename T>
__device__ __forceinline__ void fetch_block(const BlockView& bv, const T* in, long long ld, int row0,
                                            int col, int M, int N, uint4 (&v)[2]) {
  const int c = col + bv.chalf * 8;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r = row0 + bv.crow[t];
    v[t] = make_uint4(0u, 0u, 0u, 0u);
    if (r < M && c < N) v[t] = *reinterpret_cast<const uint4*>(in + static_cast<long long>(r) * ld + c);
  }
}
// Second half: through the staging block into the row view. The caller places a
// __syncwarp() between spill_block and read_row.
__device__ __forceinline__ void spill_block(const BlockView& bv, uint32_t buf, const uint4 (&v)[2]) {
  st_shared_v4(buf + bv.co[0], v[0]);
  st_shared_v4(buf + bv.co[1], v[1]);
}
__device__ __forceinline__ void read_row(const BlockView& bv, uint32_t buf, uint4& lo, uint4& hi) {
  lo = ld_shared_v4(buf + bv.row_lo);
  hi = ld_shared_v4(buf + bv.row_hi);
}

// The output matrices of a launch as TMA sees them (store and gate/up epilogues).
struct OutMaps {
  const CUtensorMap* o0;
  const CUtensorMap* o1;
  const CUtensorMap* o2;
};

// Epilogue of one 128-row accumulator tile, executed by one warp for its 32 TMEM
// lanes and its part of the tile's columns: lane i owns output row row0 + i. `taddr`
// addresses (lane quarter, first accumulator column of the tile); `stage` is the warp's
// staging area.
// ACTC: the gate activation as a compile-time constant, or -1 to read it from the
// arguments. The unrolled epilogues hold many copies of the activation per tile pass;
// with the seven-way switch in each copy the taken path is islands in a sea of
// instructions, so the usual activation (SiLU) gets a body of its own.
// Asynchronous copy of this lane's two 16-byte pieces (coalesced view) of the [32 x 16] block at
// (row0, col) of `in` into the staging block `buf`; zeros where the block leaves the matrix.
template <typename T>
__device__ __forceinline__ void fetch_block_async(const BlockView& bv, uint32_t buf, const T* in, long long ld,
                                                  int row0, int col, int M, int N) {
  const int c = col + bv.chalf * 8;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r = row0 + bv.crow[t];
    const bool ok = r < M && c < N;
    cp_async_16_zfill(buf + bv.co[t], ok ? static_cast<const void*>(in + static_cast<long long>(r) * ld + c)
                                         : static_cast<const void*>(in), ok ? 16u : 0u);
  }
}

// DHIDDEN only: next_row0 / next_n0 locate this warp's rows and the first column of the NEXT tile
// (next_row0 < 0: there is none); its first two units are requested at the end of this tile.
template <int BN, int EPI, typename T, int ACTC>
__device__ __forceinline__ void epilogue_tile16(const GemmArgs& args, const OutMaps& maps, uint32_t taddr,
                                                int row0, int lane, int batch, int n0, int part,
                                                const BlockView& bv, uint32_t stage, const T* bias0,
                                                const T* bias1, bool drop_on, int next_row0, int next_n0) {
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const int row = row0 + lane;
  const bool row_ok = row < args.M;
  const int M = args.M, N = args.N;

  if constexpr (EPI == EPI_STORE) {
    constexpr int WCOLS = TILE_N / EPI_PARTS;  // columns per warp
    static_assert(WCOLS == 64, "the store epilogue stages [32 x 64] blocks (128-byte rows)");
    const int col = n0 + part * WCOLS;
    if (col >= N || row0 >= M) return;  // warp-uniform: nothing of this block is inside the matrix
    const T* const res =
        args.in0 ? static_cast<const T*>(args.in0) + static_cast<long long>(row) * args.ld_in : nullptr;
    // the block may still be feeding the previous tile's store
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t acc[32];
      tmem_ld_32x32(taddr + part * WCOLS + hh * 32, acc);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gc = col + hh * 32 + j * 8;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[j * 8 + i]);
        if (gc < N) {
          if (bias0) {
            float b[8];
            load8(bias0 + gc, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] += b[i];
          }
          if (res && row_ok) {
            float b[8];
            load8(res + gc, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] += b[i];
          }
        }
        st_shared_v4(stage + staged_chunk<128>(lane, hh * 4 + j), pack8<T>(v));
      }
    }
    const int owner = args.push_world > 0 ? row0 / args.push_rows : -1;
    if (owner >= 0 && owner != args.push_rank) {
      // another rank's rows: the staged block leaves with plain 16-byte stores into that rank's inbox,
      // eight lanes per 128-byte row (the sum kernel that follows on every rank raises the flags)
      __syncwarp();
      const unsigned int call = __ldcg(args.push_epoch) + 1u;
      T* const dst = reinterpret_cast<T*>(args.push_base[owner] + (call & 1u) * args.push_parity_bytes);
      const int c8 = lane & 7;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        const uint4 q = ld_shared_v4(stage + staged_chunk<128>(r, c8));
        const int gr = row0 + r, gc = col + c8 * 8;
        if (gr < M && gc < N) *reinterpret_cast<uint4*>(dst + static_cast<long long>(gr) * args.ld_out + gc) = q;
      }
      __syncwarp();  // the block is free again
    } else {
      fence_proxy_async_smem();  // the staged rows become visible to the TMA engine
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(batch ? maps.o1 : maps.o0, stage, col, row0);
        bulk_commit_group();
      }
    }
  } else if constexpr (EPI == EPI_SWIGLU) {
    constexpr int WCOLS = TILE_N / EPI_PARTS;  // hidden columns per warp
    static_assert(WCOLS == 32, "the gate/up epilogue stages [32 x 32] blocks (64-byte rows)");
    const int col = n0 + part * WCOLS;
    if (col >= N || row0 >= M) return;  // warp-uniform
    const bool save = args.out1 != nullptr;  // keep the pre-activations for the backward pass
    const uint32_t buf_a = stage, buf_b = stage + STORE_STAGE_BYTES / 2;
    const long long grow = args.drop.row0_global + row;
    const bool scaled = args.row_scale != nullptr;
    const float rsv = (scaled && row_ok) ? args.row_scale[row] : 1.0f;
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
    uint4 qu[4];  // U waits in registers until H has left its block
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t rg[16], ru[16];
      tmem_ld_32x16(taddr + part * WCOLS + hh * 16, rg);
      tmem_ld_32x16(taddr + TILE_N + part * WCOLS + hh * 16, ru);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int gc = col + hh * 16 + j * 8;
        float g[8], u[8], h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          g[i] = __uint_as_float(rg[j * 8 + i]);
          u[i] = __uint_as_float(ru[j * 8 + i]);
        }
        if (scaled) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            g[i] *= rsv;
            u[i] *= rsv;
          }
        }
        if (gc < N) {
          if (bias0) {
            float b[8];
            load8(bias0 + gc, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] += b[i];
          }
          if (bias1) {
            float b[8];
            load8(bias1 + gc, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) u[i] += b[i];
          }
        }
        const uint32_t off = staged_chunk<64>(lane, hh * 2 + j);
        if (save) {
          st_shared_v4(buf_b + off, pack8<T>(g));
          qu[hh * 2 + j] = pack8<T>(u);
        }
        if (ACTC == ACT_SILU) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const f32x2 g2 = f2_pack(g[i], g[i + 1]);
            const f32x2 h2 = f2_mul(f2_mul(g2, sigmoid2(g2)), f2_pack(u[i], u[i + 1]));
            f2_unpack(h2, h[i], h[i + 1]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] = act_value(ACTC >= 0 ? ACTC : args.act, g[i]) * u[i];
        }
        if (drop_on) {
          float f[8];
          dropout_factors8_fast(args.drop, grow, args.drop.col0_global + gc, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] *= f[i];
        }
        st_shared_v4(buf_a + off, pack8<T>(h));
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(maps.o0, buf_a, col, row0);
      bulk_commit_group();
      if (save) {
        tma_store_2d(maps.o1, buf_b, col, row0);
        bulk_commit_group();
        bulk_wait_group_read<1>();  // H has been read out of its block
      }
    }
    if (save) {
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) st_shared_v4(buf_a + staged_chunk<64>(lane, c), qu[c]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(maps.o2, buf_a, col, row0);
        bulk_commit_group();
      }
    }
  } else {  // EPI_DHIDDEN
    constexpr int NU = TILE_N / 16 / EPI_PARTS;  // 16-column units per warp
    static_assert(NU >= 2 && NU % 2 == 0, "units alternate between the warp's two pairs of staging blocks");
    const int u0 = part * NU;
    T* const out_g = static_cast<T*>(args.out0);
    T* const out_u = static_cast<T*>(args.out1);
    const T* const in_g = static_cast<const T*>(args.in0);
    const T* const in_u = static_cast<const T*>(args.in1);
    const long long grow = args.drop.row0_global + row;
#pragma unroll
    for (int ui = 0; ui < NU; ++ui) {
      const int col = n0 + (u0 + ui) * 16;
      const uint32_t buf_g = stage + (ui & 1) * (2 * BLK_BYTES), buf_u = buf_g + BLK_BYTES;
      uint32_t acc[16];
      tmem_ld_32x16(taddr + (u0 + ui) * 16, acc);
      // this unit's G and U were requested two units ago; the request after it may still be in flight
      cp_async_wait_group<1>();
      __syncwarp();
      uint4 gq[2], uq[2];
      read_row(bv, buf_g, gq[0], gq[1]);
      read_row(bv, buf_u, uq[0], uq[1]);
      tmem_ld_wait();
      uint4 qg[2], qu[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int gc = col + j * 8;
        float dh[8], g[8], u[8], dg[8], du[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) dh[i] = __uint_as_float(acc[j * 8 + i]);
        unpack8<T>(gq[j], g);
        unpack8<T>(uq[j], u);
        if (drop_on) {
          float f[8];
          dropout_factors8_fast(args.drop, grow, args.drop.col0_global + gc, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) dh[i] *= f[i];
        }
        if (ACTC == ACT_SILU) {
          // s = sigma(g), f = g s, f' = s + f (1 - s); d_up = dh f, d_gate = dh u f'
          const f32x2 one = f2_pack(1.0f, 1.0f), neg = f2_pack(-1.0f, -1.0f);
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const f32x2 g2 = f2_pack(g[i], g[i + 1]), dh2 = f2_pack(dh[i], dh[i + 1]);
            const f32x2 s2 = sigmoid2(g2);
            const f32x2 f2v = f2_mul(g2, s2);
            const f32x2 df2 = f2_fma(f2v, f2_fma(s2, neg, one), s2);
            f2_unpack(f2_mul(dh2, f2v), du[i], du[i + 1]);
            f2_unpack(f2_mul(f2_mul(dh2, f2_pack(u[i], u[i + 1])), df2), dg[i], dg[i + 1]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float f, df;
            act_value_grad(ACTC >= 0 ? ACTC : args.act, g[i], f, df);
            du[i] = dh[i] * f;
            dg[i] = dh[i] * u[i] * df;
          }
        }
        qg[j] = pack8<T>(dg);
        qu[j] = pack8<T>(du);
      }
      // In place: each lane overwrites the row it has just read, then the block leaves in
      // the coalesced view.
      store_block<T>(bv, buf_g, out_g, args.ld_out, row0, col, M, N, qg[0], qg[1]);
      store_block<T>(bv, buf_u, out_u, args.ld_out, row0, col, M, N, qu[0], qu[1]);
      __syncwarp();  // the pair has been read out: request the unit after next into it
      if (ui + 2 < NU) {
        fetch_block_async<T>(bv, buf_g, in_g, args.ld_in, row0, col + 32, M, N);
        fetch_block_async<T>(bv, buf_u, in_u, args.ld_in, row0, col + 32, M, N);
      } else if (next_row0 >= 0) {
        const int ncol = next_n0 + (u0 + ui + 2 - NU) * 16;
        fetch_block_async<T>(bv, buf_g, in_g, args.ld_in, next_row0, ncol, M, N);
        fetch_block_async<T>(bv, buf_u, in_u, args.ld_in, next_row0, ncol, M, N);
      }
      cp_async_commit();  // one group per unit, empty when there was nothing left to request
    }
  }
}

// fp32 matrices (tf32 products): the store and gate/up epilogues for 4-byte outputs. A warp's
// staging area holds one [32 rows x 32 columns] fp32 block (128-byte rows), so the plain store
// sends its 64 columns as two blocks and the training gate/up kernel sends H, G and U one after
// the other (re-reading the accumulators, which stay in TMEM until the tile is handed back).
// This is the compatibility path for fp32 modules, not a tuned one.
__device__ __forceinline__ void stage_store_f32(const CUtensorMap* map, uint32_t stage, int lane, int col, int row0,
                                                const float (&v)[32]) {
  if (lane == 0) bulk_wait_group_read<0>();  // the block may still feed the previous store
  __syncwarp();
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = __float_as_uint(v[4 * c]);
    q.y = __float_as_uint(v[4 * c + 1]);
    q.z = __float_as_uint(v[4 * c + 2]);
    q.w = __float_as_uint(v[4 * c + 3]);
    st_shared_v4(stage + staged_chunk<128>(lane, c), q);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map, stage, col, row0);
    bulk_commit_group();
  }
}

template <int BN, int EPI, int ACTC>
__device__ __forceinline__ void epilogue_tile_f32(const GemmArgs& args, const OutMaps& maps, uint32_t taddr,
                                                  int row0, int lane, int batch, int n0, int part, uint32_t stage,
                                                  const float* bias0, const float* bias1, bool drop_on) {
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const int row = row0 + lane;
  const bool row_ok = row < args.M;
  const int M = args.M, N = args.N;
  auto add8 = [&](const float* p, int gc, float* v) {  // v[0..8) += p[gc..gc+8) where inside the matrix
    if (p != nullptr && gc < N) {
      float b[8];
      load8(p + gc, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += b[i];
    }
  };
  if constexpr (EPI == EPI_STORE) {
    constexpr int WCOLS = TILE_N / EPI_PARTS;
    const int col = n0 + part * WCOLS;
    if (col >= N || row0 >= M) return;
    const float* const res =
        (args.in0 && row_ok) ? static_cast<const float*>(args.in0) + static_cast<long long>(row) * args.ld_in : nullptr;
#pragma unroll
    for (int hh = 0; hh < WCOLS / 32; ++hh) {
      if (col + hh * 32 >= N) break;  // warp-uniform
      uint32_t acc[32];
      tmem_ld_32x32(taddr + part * WCOLS + hh * 32, acc);
      tmem_ld_wait();
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        add8(bias0, col + hh * 32 + j * 8, v + 8 * j);
        add8(res, col + hh * 32 + j * 8, v + 8 * j);
      }
      stage_store_f32(batch ? maps.o1 : maps.o0, stage, lane, col + hh * 32, row0, v);
    }
  } else {  // EPI_SWIGLU
    constexpr int WCOLS = TILE_N / EPI_PARTS;
    static_assert(WCOLS == 32, "one [32 x 32] fp32 block per warp");
    const int col = n0 + part * WCOLS;
    if (col >= N || row0 >= M) return;
    const bool save = args.out1 != nullptr;
    const long long grow = args.drop.row0_global + row;
    const float rsv = (args.row_scale != nullptr && row_ok) ? args.row_scale[row] : 1.0f;
    // what: 0 = H (activation, product, dropout), 1 = G, 2 = U; sixteen columns at a time
    auto emit = [&](const CUtensorMap* map, int what) {
      if (lane == 0) bulk_wait_group_read<0>();  // the block may still feed the previous store
      __syncwarp();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t rg[16], ru[16];
        if (what != 2) tmem_ld_32x16(taddr + part * WCOLS + hh * 16, rg);
        if (what != 1) tmem_ld_32x16(taddr + TILE_N + part * WCOLS + hh * 16, ru);
        tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int gc = col + hh * 16 + j * 8;
          float g[8], u[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            g[i] = what != 2 ? __uint_as_float(rg[j * 8 + i]) * rsv : 0.f;
            u[i] = what != 1 ? __uint_as_float(ru[j * 8 + i]) * rsv : 0.f;
          }
          if (what != 2) add8(bias0, gc, g);
          if (what != 1) add8(bias1, gc, u);
          if (what == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] = act_value(ACTC >= 0 ? ACTC : args.act, g[i]) * u[i];
            if (drop_on) {
              float f[8];
              dropout_factors8_fast(args.drop, grow, args.drop.col0_global + gc, f);
#pragma unroll
              for (int i = 0; i < 8; ++i) g[i] *= f[i];
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) v[j * 8 + i] = what == 2 ? u[i] : g[i];
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 q;
          q.x = __float_as_uint(v[4 * c]);
          q.y = __float_as_uint(v[4 * c + 1]);
          q.z = __float_as_uint(v[4 * c + 2]);
          q.w = __float_as_uint(v[4 * c + 3]);
          st_shared_v4(stage + staged_chunk<128>(lane, hh * 4 + c), q);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map, stage, col, row0);
        bulk_commit_group();
      }
    };
    if (save) {
      emit(maps.o1, 1);
      emit(maps.o2, 2);
    }
    emit(maps.o0, 0);
  }
}

template <int BN, int EPI, typename T, int ACTC>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& args, const OutMaps& maps, uint32_t taddr,
                                              int row0, int lane, int batch, int n0, int part,
                                              const BlockView& bv, uint32_t stage, const T* bias0,
                                              const T* bias1, bool drop_on, int next_row0, int next_n0) {
  if constexpr (sizeof(T) == 4)
    epilogue_tile_f32<BN, EPI, ACTC>(args, maps, taddr, row0, lane, batch, n0, part, stage, bias0, bias1, drop_on);
  else
    epilogue_tile16<BN, EPI, T, ACTC>(args, maps, taddr, row0, lane, batch, n0, part, bv, stage, bias0, bias1,
                                      drop_on, next_row0, next_n0);
}

// Row sums of this CTA's 128 rows of the MN-major A operand over the tile's SHARE of the
// reduction blocks (block kb belongs to the column tile kb mod n_tiles of its row tile, so
// the column tiles of one row tile divide the work between them), by the watcher warp while
// the main loop runs: the blocks are fetched with TMA through the same tensor map the
// producer uses into a private ring in the epilogue's staging area (idle at that time),
// summed from shared memory, and the partial sums go to `asum_part`. The CTA that brings
// the count of a 128-row block to n_tiles adds the partials in column-tile order (so the
// result does not depend on arrival order) and writes the sums.
//   seq      running number of this warp's ring loads (ring slot and mbarrier phase follow from it)
//   returns false if a wait ran out
template <typename T>
__device__ __forceinline__ bool asum_tile(const GemmArgs& args, const CUtensorMap* map, const TileCoord& tc,
                                          int lane, int n_tiles, int mn0, int mn_pad, uint32_t ring,
                                          uint32_t bar0, uint32_t& seq, volatile int* abortp) {
  constexpr uint32_t BUF_BYTES = 2 * BK * 128;  // two [64 reduction rows x 64 columns] boxes
  const int count = tc.n_tile < args.kb0 ? (args.kb0 - tc.n_tile + n_tiles - 1) / n_tiles : 0;
  auto issue = [&](int i) {  // lane 0
    const uint32_t slot = (seq + i) % ASUM_BUFS;
    const uint32_t dst = ring + slot * BUF_BYTES, bar = bar0 + 8u * slot;
    const int k0 = (tc.n_tile + i * n_tiles) * BK;
    fence_proxy_async_smem();
    mbar_expect_tx(bar, BUF_BYTES);
    tma_load_2d(dst, map, bar, mn0, k0);
    tma_load_2d(dst + BK * 128, map, bar, mn0 + 64, k0);
  };
  if (lane == 0)
    for (int i = 0; i < count && i < ASUM_BUFS; ++i) issue(i);
  const int j = lane & 7, rg = lane >> 3;  // 16-byte chunk (8 columns) and row group of this lane
  float acc[2][8];
#pragma unroll
  for (int b = 0; b < 2; ++b)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[b][c] = 0.f;
  bool ok = true;
  for (int i = 0; i < count; ++i) {
    const uint32_t slot = (seq + i) % ASUM_BUFS, phase = ((seq + i) / ASUM_BUFS) & 1u;
    ok = mbar_wait_warp(bar0 + 8u * slot, phase, abortp, lane);
    if (!ok) break;
    const uint32_t buf = ring + slot * BUF_BYTES;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
#pragma unroll 4
      for (int r = rg; r < BK; r += 4) {
        float v[8];
        unpack8<T>(ld_shared_v4(buf + b * (BK * 128) + staged_chunk<128>(r, j)), v);
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[b][c] += v[c];
      }
    }
    __syncwarp();  // every lane has read the slot before it is refilled
    if (lane == 0 && i + ASUM_BUFS < count) issue(i + ASUM_BUFS);
  }
  seq += static_cast<uint32_t>(count);
  if (!ok) return false;
  // lanes with the same chunk hold different rows: fold them onto lanes 0..7
#pragma unroll
  for (int b = 0; b < 2; ++b)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      acc[b][c] += __shfl_xor_sync(0xffffffffu, acc[b][c], 8);
      acc[b][c] += __shfl_xor_sync(0xffffffffu, acc[b][c], 16);
    }
  float* const part = args.asum_part + (static_cast<long long>(tc.batch) * n_tiles + tc.n_tile) * mn_pad + mn0;
  if (lane < 8) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      float4* q = reinterpret_cast<float4*>(part + 64 * b + 8 * j);
      q[0] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
      q[1] = make_float4(acc[b][4], acc[b][5], acc[b][6], acc[b][7]);
    }
  }
  __threadfence();
  __syncwarp();
  int last = 0;
  int* const cnt = args.asum_cnt + static_cast<long long>(tc.batch) * (mn_pad / 128) + mn0 / 128;
  if (lane == 0) {
    last = atomicAdd(cnt, 1) == n_tiles - 1 ? 1 : 0;
    if (last) *cnt = 0;  // nobody else touches this counter again in this launch
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (last) {
    __threadfence();
    T* const out = static_cast<T*>(args.asum_out[tc.batch]);
    const float* const p0 = args.asum_part + static_cast<long long>(tc.batch) * n_tiles * mn_pad + mn0;
    // 128 columns, 4 per lane
    const int c = lane * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = 0; t < n_tiles; ++t) {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(p0 + static_cast<long long>(t) * mn_pad + c));
      s.x += q.x; s.y += q.y; s.z += q.z; s.w += q.w;
    }
    if (mn0 + c < args.M) {  // M is a multiple of 8: the four columns are inside or outside together
      uint2 o;
      o.x = Pack2<T>::pack(s.x, s.y);
      o.y = Pack2<T>::pack(s.z, s.w);
      *reinterpret_cast<uint2*>(out + mn0 + c) = o;
    }
  }
  return true;
}

// The watcher role (warp 18, all lanes): for every tile of this CTA, wait until the MMA
// issuer's commit has marked the accumulator full, publish the verdict and release the
// epilogue warps from their named barrier. It arrives on the barrier whatever the
// outcome, so the epilogue warps always wake up, read the same verdict and leave together.
// ASUM: before that wait it takes the tile's share of the A operand's row sums (asum_tile),
// using the staging area between the previous tile's epilogue and this tile's.
// NSUB = 2 (wide tiles, see the pair kernel): one accumulator buffer instead of two.
template <typename T, int TILE_M, bool ASUM, int NSUB = 1>
__device__ __forceinline__ void watcher_role(const GemmArgs& args, const CUtensorMap* mapA0,
                                             const CUtensorMap* mapA1, int lane, int first_tile,
                                             int tile_stride, int total_tiles, int m_tiles, int n_tiles,
                                             int row_off, uint32_t tfull0, uint32_t asum_bar0,
                                             uint32_t epi_smem, volatile int* epi_go, int* abort_flag) {
  volatile int* abortp = abort_flag;
  int local = 0;
  uint32_t seq = 0;
  for (int tile = first_tile; tile < total_tiles; tile += tile_stride, ++local) {
    const int acc = NSUB == 2 ? 0 : (local & 1);
    const uint32_t acc_parity = NSUB == 2 ? (local & 1) : ((local >> 1) & 1);
    bool ok = true;
    if constexpr (ASUM) {
      const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
      const int mn0 = tc.m_tile * TILE_M + row_off;
      if (local > 0) named_bar_sync(EPI_DONE_BAR, EPI_BAR_THREADS);  // the staging area is free
      if (args.asum_out[tc.batch] != nullptr && mn0 < args.M)
        ok = asum_tile<T>(args, tc.batch ? mapA1 : mapA0, tc, lane, n_tiles, mn0, m_tiles * TILE_M, epi_smem,
                          asum_bar0, seq, abortp);
    }
    ok = mbar_wait_warp<WATCHER_SLEEP_NS>(tfull0 + 8u * acc, acc_parity, abortp, lane) && ok;
    tc_fence_after_sync();
    if (lane == 0) {
      epi_go[acc] = ok ? 1 : 0;
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
      }
    }
    tc_fence_before_sync();
    __syncwarp();
    named_bar_arrive(EPI_BAR_ID0 + acc, EPI_BAR_THREADS);
    if (!ok) break;
  }
}

// The epilogue role of one warp for all tiles of its CTA (or CTA pair).
//   TILE_M     rows per tile: 128, or 256 for a CTA pair (row_off = cluster rank * 128)
//   tempty0    shared::cta address of tempty[0] ([1] is 8 bytes on)
//   REMOTE     tempty lives in the pair's leader CTA: arrive through the cluster
//   epi_smem   this CTA's epilogue staging area
//   NSUB       accumulator sub-tiles of BN columns per tile (2 = wide tiles, one accumulator buffer)
template <int BN, int EPI, typename T, int TILE_M, bool REMOTE, bool ASUM, int NSUB = 1>
__device__ __forceinline__ void epilogue_role(const GemmArgs& args, const OutMaps& maps, int warp,
                                              int lane, int first_tile, int tile_stride,
                                              int total_tiles, int m_tiles, int n_tiles, int row_off,
                                              uint32_t tmem_base, uint32_t tempty0, uint32_t epi_smem,
                                              volatile int* epi_go) {
  static_assert(NSUB == 1 || EPI == EPI_STORE, "wide tiles are for the plain store");
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : NSUB * BN;
  const int ew = warp - 2;       // epilogue warp index 0..15
  const int quarter = warp & 3;  // TMEM lanes this warp may read
  const int col_part = ew >> 2;
  const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
  const T* const bias0 = static_cast<const T*>(args.bias0);
  const T* const bias1 = static_cast<const T*>(args.bias1);
  const bool drop_on = args.drop.thresh != 0u;
  const BlockView bv(lane);
  const uint32_t stage = epi_smem + ew * STORE_STAGE_BYTES;
  if constexpr (EPI == EPI_DHIDDEN) {
    // the first tile's first two units; every later request is made from inside epilogue_tile
    if (first_tile < total_tiles) {
      const TileCoord t0 = decode_tile(first_tile, m_tiles, n_tiles, args.group_m);
      const int r0 = t0.m_tile * TILE_M + row_off + quarter * 32;
      const int c0 = t0.n_tile * TILE_N + col_part * (TILE_N / EPI_PARTS);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint32_t buf = stage + q * (2 * BLK_BYTES);
        fetch_block_async<T>(bv, buf, static_cast<const T*>(args.in0), args.ld_in, r0, c0 + 16 * q, args.M, args.N);
        fetch_block_async<T>(bv, buf + BLK_BYTES, static_cast<const T*>(args.in1), args.ld_in, r0, c0 + 16 * q,
                             args.M, args.N);
        cp_async_commit();
      }
    }
  }
  int local = 0;
  for (int tile = first_tile; tile < total_tiles; tile += tile_stride, ++local) {
    const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
    int next_row0 = -1, next_n0 = 0;
    if (EPI == EPI_DHIDDEN && tile + tile_stride < total_tiles) {
      const TileCoord nx = decode_tile(tile + tile_stride, m_tiles, n_tiles, args.group_m);
      next_row0 = nx.m_tile * TILE_M + row_off + quarter * 32;
      next_n0 = nx.n_tile * TILE_N;
    }
    const int acc = NSUB == 2 ? 0 : (local & 1);
    __syncwarp();
    named_bar_sync(EPI_BAR_ID0 + acc, EPI_BAR_THREADS);  // asleep until the watcher arrives
    if (epi_go[acc] == 0) break;                         // the same verdict for all sixteen warps
    tc_fence_after_sync();
    const uint32_t taddr = tmem_base + (NSUB == 2 ? 0 : acc * BN) + lane_addr;
    const int row0 = tc.m_tile * TILE_M + row_off + quarter * 32;
    if (EPI != EPI_STORE && args.act == ACT_SILU) {
      epilogue_tile<BN, EPI, T, ACT_SILU>(args, maps, taddr, row0, lane, tc.batch, tc.n_tile * TILE_N, col_part, bv,
                                          stage, bias0, bias1, drop_on, next_row0, next_n0);
    } else {
#pragma unroll
      for (int sub = 0; sub < NSUB; ++sub)  // a wide tile leaves as NSUB tiles of BN columns
        epilogue_tile<BN, EPI, T, -1>(args, maps, taddr + sub * BN, row0, lane, tc.batch,
                                      tc.n_tile * TILE_N + sub * BN, col_part, bv, stage, bias0, bias1, drop_on,
                                      next_row0, next_n0);
    }
    // Every tcgen05.ld of this tile was followed by tcgen05.wait::ld, so the data is in
    // registers: hand the TMEM buffer back to the MMA issuer. The arrive has release
    // semantics; no fence is placed here on purpose, since a fence would also wait for
    // this warp's outstanding global stores.
    __syncwarp();
    if (lane == 0) {
      if (REMOTE) mbar_arrive_cluster(mapa_shared(tempty0 + 8u * acc, 0));
      else mbar_arrive(tempty0 + 8u * acc);
    }
    if (ASUM && tile + tile_stride < total_tiles) {
      // The watcher borrows the staging area until the next tile's epilogue: tell it once
      // this warp's stores have been read out of it.
      if (lane == 0) bulk_wait_group_read<0>();
      __syncwarp();
      named_bar_arrive(EPI_DONE_BAR, EPI_BAR_THREADS);
    }
  }
  // Shared memory must outlive the TMA stores that still read it (and the dH epilogue's last,
  // empty, copy groups must have retired).
  if (EPI != EPI_DHIDDEN && lane == 0) bulk_wait_group_read<0>();
  if (EPI == EPI_DHIDDEN) cp_async_wait_group<0>();
}

// ------------------------------------------------------------------ kernel --
template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES, bool ASUM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA0,
                    const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CUtensorMap tmO0,
                    const __grid_constant__ CUtensorMap tmO1,
                    const __grid_constant__ CUtensorMap tmO2, const GemmArgs args) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "tcgen05 N range for M = 128");
  static_assert(!(EPI == EPI_SWIGLU) || (BN == 256 && !B_MN), "gate|up tile is 128 + 128 rows");
  static_assert(!B_MN || BN % 64 == 0, "MN-major B arrives in 64-column boxes");
  static_assert(!ASUM || (A_MN && EPI == EPI_STORE), "row sums are taken of an MN-major A beside a plain store");
  static_assert(sizeof(T) == 2 || (!A_MN && !B_MN && EPI != EPI_DHIDDEN),
                "fp32 (tf32) operands: K-major only, store and gate/up epilogues only");
  constexpr uint32_t A_BYTES = BM * 128;
  constexpr uint32_t B_BYTES = BN * 128;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = tmem_cols_for(BN);
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;  // output columns per tile
  // Descriptor geometry (bytes). K-major: rows of 128 B, 8-row groups 1024 B apart,
  // 32 B per UMMA_K step. MN-major: 64-wide chunks of BK rows (8 KB apart), 8
  // reduction rows per 1024 B group, 2 groups (2048 B) per UMMA_K step.
  constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, B_LBO = B_MN ? BK * 128 : 16;
  constexpr uint32_t A_KSTEP = (A_MN ? 2048 : 32) >> 4, B_KSTEP = (B_MN ? 2048 : 32) >> 4;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4 + ASUM_BUFS];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ volatile int epi_go[2];

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (args.M + BM - 1) / BM;
  const int n_tiles = (args.N + TILE_N - 1) / TILE_N;
  const int total_tiles = args.batches * m_tiles * n_tiles;
  const int kb_total = args.kb0 + args.kb1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    epi_go[0] = epi_go[1] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < ASUM_BUFS; ++b) mbar_init(bar_base + 8u * (2 * STAGES + 4 + b), 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EPI_WARPS);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB0);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
        const int m0 = tc.m_tile * BM;
        const int n0 = tc.n_tile * TILE_N;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait<PRODUCER_SLEEP_NS>(empty_bar(stage), phase ^ 1u, abortp)) {
            ok = false;
            break;
          }
          const int seg = kb >= args.kb0 ? 1 : 0;
          const int k0 = (seg ? kb - args.kb0 : kb) * row_elems<T>();
          const CUtensorMap* ma = (seg | tc.batch) ? &tmA1 : &tmA0;
          const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, STAGE_BYTES);
          if (A_MN) {
            tma_load_2d(sa, ma, fb, m0, k0);
            tma_load_2d(sa + BK * 128, ma, fb, m0 + 64, k0);
          } else {
            tma_load_2d(sa, ma, fb, k0, m0);
          }
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(sb, &tmB0, fb, k0, n0);
            tma_load_2d(sb + (BN / 2) * 128, &tmB1, fb, k0, n0);
          } else if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), mb, fb, n0 + 64 * j, k0);
          } else {
            tma_load_2d(sb, mb, fb, k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_PRODUCER);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abortp)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa, A_LBO, 1024);
          const uint64_t bdesc = make_smem_desc(sa + A_BYTES, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (sizeof(T) == 4)
              umma_tf32(d_tmem, adesc + static_cast<uint64_t>(k * A_KSTEP),
                        bdesc + static_cast<uint64_t>(k * B_KSTEP), args.idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16(d_tmem, adesc + static_cast<uint64_t>(k * A_KSTEP),
                       bdesc + static_cast<uint64_t>(k * B_KSTEP), args.idesc,
                       (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_MMA);
      }
    }
  } else if (warp == WATCHER_WARP) {
    watcher_role<T, BM, ASUM>(args, &tmA0, &tmA1, lane, blockIdx.x, gridDim.x, total_tiles, m_tiles, n_tiles, 0,
                              tfull_bar(0), bar_base + 8u * (2 * STAGES + 4), smem_base + STAGES * STAGE_BYTES,
                              epi_go, &abort_flag);
  } else {
    // ------------------------------------------------------------ epilogue --
    const OutMaps maps{&tmO0, &tmO1, &tmO2};
    epilogue_role<BN, EPI, T, BM, false, ASUM>(args, maps, warp, lane, blockIdx.x, gridDim.x, total_tiles, m_tiles,
                                         n_tiles, 0, tmem_base, tempty_bar(0),
                                         smem_base + STAGES * STAGE_BYTES, epi_go);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------- CTA-pair kernel ----
// Same roles and pipeline as above, but two CTAs on neighbouring SMs (a cluster
// of 2) work on one 256-row tile with tcgen05.mma.cta_group::2: each CTA stages
// its own 128 rows of A and its own half of B's columns, so a CTA fetches
// 128 x 64 of A plus (BN/2) x 64 of B per reduction block instead of 128 x 64 plus
// BN x 64. That cuts the L2 -> shared-memory traffic per MMA by a third at BN = 256,
// which is what bounds the single-CTA kernel. No TMA multicast is involved: every
// byte of shared memory is written by the CTA that owns it.
//
// Protocol differences to the single-CTA kernel:
//   full[s]    lives in the leader (cluster rank 0); both CTAs' loads count their
//              bytes on it; the leader's producer arms it for 2 x the per-CTA bytes.
//   empty[s], tfull[a]   exist in both CTAs; the leader's MMA thread commits to
//              both copies at once.
//   tempty[a]  lives in the leader, 32 arrivals: the 16 epilogue warps of each CTA.
//
// NSUB = 2, "wide tiles" (plain store only): the pair computes a 256 x 512 tile with two N = 256 MMAs per
// reduction step that share A, so 96 KB of operands cross from L2 per 256 x 512 x 64 block instead of 128 KB
// (the GEMMs are bound by that stream). The accumulator then fills all 512 TMEM columns: there is one buffer,
// the epilogue of a tile does not overlap the next tile's main loop, and the ring has 3 stages of 48 KB. Pays
// where the reduction is long (the epilogue is a few percent of a tile).
template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES, bool ASUM, int NSUB = 1>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA0,
                         const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmB0,
                         const __grid_constant__ CUtensorMap tmB1,
                         const __grid_constant__ CUtensorMap tmO0,
                         const __grid_constant__ CUtensorMap tmO1,
                         const __grid_constant__ CUtensorMap tmO2, const GemmArgs args) {
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tcgen05 N range for M = 256");
  static_assert(!(EPI == EPI_SWIGLU) || (BN == 256 && !B_MN), "gate|up tile is 128 + 128 rows");
  static_assert(!B_MN || BN % 128 == 0, "MN-major B arrives in 64-column boxes per CTA");
  static_assert(!ASUM || (A_MN && EPI == EPI_STORE), "row sums are taken of an MN-major A beside a plain store");
  static_assert(sizeof(T) == 2 || (!A_MN && !B_MN && EPI != EPI_DHIDDEN),
                "fp32 (tf32) operands: K-major only, store and gate/up epilogues only");
  constexpr int HALF_N = BN / 2;  // B columns staged by each CTA
  constexpr uint32_t A_BYTES = BM * 128;
  constexpr uint32_t B_BYTES = HALF_N * 128;
  static_assert(NSUB == 1 || (NSUB == 2 && BN == 256 && EPI == EPI_STORE), "wide tiles: 2 x 256 columns");
  constexpr uint32_t STAGE_BYTES = A_BYTES + NSUB * B_BYTES;
  constexpr uint32_t TMEM_COLS = NSUB == 2 ? 512 : tmem_cols_for(BN);
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : NSUB * BN;
  constexpr int PAIR_M = 2 * BM;
  constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, B_LBO = B_MN ? BK * 128 : 16;
  constexpr uint32_t A_KSTEP = (A_MN ? 2048 : 32) >> 4, B_KSTEP = (B_MN ? 2048 : 32) >> 4;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4 + ASUM_BUFS];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ volatile int epi_go[2];

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int m_tiles = (args.M + PAIR_M - 1) / PAIR_M;
  const int n_tiles = (args.N + TILE_N - 1) / TILE_N;
  const int total_tiles = args.batches * m_tiles * n_tiles;
  const int kb_total = args.kb0 + args.kb1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    epi_go[0] = epi_go[1] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < ASUM_BUFS; ++b) mbar_init(bar_base + 8u * (2 * STAGES + 4 + b), 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * EPI_WARPS);  // the epilogue warps of both CTAs of the pair
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB0);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_base_holder), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
        const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
        const int m0 = tc.m_tile * PAIR_M + static_cast<int>(rank) * BM;
        const int n0 = tc.n_tile * TILE_N;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait<PRODUCER_SLEEP_NS>(empty_bar(stage), phase ^ 1u, abortp)) {
            ok = false;
            break;
          }
          const int seg = kb >= args.kb0 ? 1 : 0;
          const int k0 = (seg ? kb - args.kb0 : kb) * row_elems<T>();
          const CUtensorMap* ma = (seg | tc.batch) ? &tmA1 : &tmA0;
          const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t fb = mapa_shared(full_bar(stage), 0);  // the leader's barrier
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          if (A_MN) {
            tma_load_2d_pair(sa, ma, fb, m0, k0);
            tma_load_2d_pair(sa + BK * 128, ma, fb, m0 + 64, k0);
          } else {
            tma_load_2d_pair(sa, ma, fb, k0, m0);
          }
          if (EPI == EPI_SWIGLU) {
            // leader stages the gate rows, the peer the up rows of the same hidden columns
            tma_load_2d_pair(sb, rank == 0 ? &tmB0 : &tmB1, fb, k0, n0);
          } else if (B_MN) {
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub)
#pragma unroll
              for (int j = 0; j < HALF_N / 64; ++j)
                tma_load_2d_pair(sb + sub * B_BYTES + j * (BK * 128), mb, fb,
                                 n0 + sub * BN + static_cast<int>(rank) * HALF_N + 64 * j, k0);
          } else {
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub)
              tma_load_2d_pair(sb + sub * B_BYTES, mb, fb, k0, n0 + sub * BN + static_cast<int>(rank) * HALF_N);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_PRODUCER);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader only) --
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++local) {
        const int acc = NSUB == 2 ? 0 : (local & 1);
        const uint32_t acc_phase = NSUB == 2 ? (local & 1) : ((local >> 1) & 1);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (NSUB == 2 ? 0 : acc * BN);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abortp)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa, A_LBO, 1024);
#pragma unroll
          for (int sub = 0; sub < NSUB; ++sub) {
            const uint64_t bdesc = make_smem_desc(sa + A_BYTES + sub * B_BYTES, B_LBO, 1024);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              if (sizeof(T) == 4)
                umma_tf32_pair(d_tmem + sub * BN, adesc + static_cast<uint64_t>(k * A_KSTEP),
                               bdesc + static_cast<uint64_t>(k * B_KSTEP), args.idesc, (kb | k) != 0 ? 1u : 0u);
              else
                umma_f16_pair(d_tmem + sub * BN, adesc + static_cast<uint64_t>(k * A_KSTEP),
                              bdesc + static_cast<uint64_t>(k * B_KSTEP), args.idesc,
                              (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit_pair(tfull_bar(acc));
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_MMA);
      }
    }
  } else if (warp == WATCHER_WARP) {
    watcher_role<T, PAIR_M, ASUM, NSUB>(args, &tmA0, &tmA1, lane, pair, num_pairs, total_tiles, m_tiles, n_tiles,
                                  static_cast<int>(rank) * BM, tfull_bar(0), bar_base + 8u * (2 * STAGES + 4),
                                  smem_base + STAGES * STAGE_BYTES, epi_go, &abort_flag);
  } else {
    // ------------------------------------------------------------ epilogue --
    const OutMaps maps{&tmO0, &tmO1, &tmO2};
    epilogue_role<BN, EPI, T, PAIR_M, true, ASUM, NSUB>(args, maps, warp, lane, pair, num_pairs, total_tiles, m_tiles,
                                            n_tiles, static_cast<int>(rank) * BM, tmem_base, tempty_bar(0),
                                            smem_base + STAGES * STAGE_BYTES, epi_go);
  }

  // Neither CTA may exit (or free TMEM) while its peer can still read its shared
  // memory, write its TMEM or arrive on its barriers.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gmlp
