// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused gated-MLP
// epilogues. One CTA per SM walks a grouped tile order; per CTA:
//   warp 0 (one lane)  TMA producer: fills a STAGES-deep shared-memory ring
//   warp 1 (one lane)  MMA issuer: tcgen05.mma into one of two TMEM accumulators
//   warps 2..5         epilogue: tcgen05.ld the finished accumulator, apply the
//                      fused elementwise work, store to global memory
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of
// tile i+1. No cluster launch and no TMA multicast is used.
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
  uint32_t idesc;
  int* status;  // device word; a role that gives up a wait stores its code here
  void* out0;
  void* out1;
  void* out2;
  const void* in0;
  const void* in1;
  const void* bias0;
  const void* bias1;
  long long ld_out;  // row pitch (elements) of out*
  long long ld_in;   // row pitch (elements) of in*
  DropoutParams drop;
};

constexpr int BM = 128;        // rows per tile = TMEM lanes
constexpr int BK = 64;         // reduction elements per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;     // reduction elements per tcgen05.mma (16-bit inputs)
constexpr int GEMM_THREADS = 192;

__host__ __device__ constexpr uint32_t tmem_cols_for(int bn) {
  return (2 * bn <= 32) ? 32u : (2 * bn <= 64) ? 64u : (2 * bn <= 128) ? 128u
         : (2 * bn <= 256) ? 256u : 512u;
}

template <int BN, int STAGES>
constexpr size_t gemm_smem_bytes() {
  return static_cast<size_t>(STAGES) * (BM * 128 + BN * 128) + 1024;
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

// sigma(x) = 1 / (1 + e^-x); the clamp keeps e^-x finite in fp32.
__device__ __forceinline__ float sigmoid_f(float x) {
  return __fdividef(1.0f, 1.0f + __expf(-fmaxf(x, -80.0f)));
}

// keep/scale factors for the 8 consecutive columns starting at (grow, gcol),
// gcol a multiple of 4 in the global index space.
__device__ __forceinline__ void dropout_factors8(const DropoutParams& d, long long grow,
                                                 long long gcol, float (&f)[8]) {
  const unsigned long long e =
      static_cast<unsigned long long>(grow) * static_cast<unsigned long long>(d.ncols_global) +
      static_cast<unsigned long long>(gcol);
  const Philox4 r0 = dropout_words(d, e >> 2);
  const Philox4 r1 = dropout_words(d, (e >> 2) + 1);
  f[0] = r0.x >= d.thresh ? d.scale : 0.0f;
  f[1] = r0.y >= d.thresh ? d.scale : 0.0f;
  f[2] = r0.z >= d.thresh ? d.scale : 0.0f;
  f[3] = r0.w >= d.thresh ? d.scale : 0.0f;
  f[4] = r1.x >= d.thresh ? d.scale : 0.0f;
  f[5] = r1.y >= d.thresh ? d.scale : 0.0f;
  f[6] = r1.z >= d.thresh ? d.scale : 0.0f;
  f[7] = r1.w >= d.thresh ? d.scale : 0.0f;
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

// Epilogue of one 128-row accumulator tile, executed by one warp for its 32 TMEM
// lanes: lane i owns output row `row` and walks the tile's columns in chunks of 32.
// `taddr` addresses (lane quarter, first accumulator column of the tile).
template <int BN, int EPI, typename T>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& args, uint32_t taddr, int row,
                                              int batch, int n0, T* out0, T* out1, T* out2,
                                              const T* in0, const T* in1, const T* bias0,
                                              const T* bias1, bool drop_on) {
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  const bool row_ok = row < args.M;
        if (EPI == EPI_STORE) {
          T* const out = (batch ? out1 : out0) + static_cast<long long>(row) * args.ld_out;
          const T* const res = in0 ? in0 + static_cast<long long>(row) * args.ld_in : nullptr;
  #pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int col = n0 + c * 32;
            if (col >= args.N) break;
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
            if (row_ok) {
  #pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int gc = col + j * 8;
                if (gc < args.N) {
                  float v[8];
  #pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[j * 8 + i]);
                  if (bias0) {
                    float b[8];
                    load8(bias0 + gc, b);
  #pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] += b[i];
                  }
                  if (res) {
                    float b[8];
                    load8(res + gc, b);
  #pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] += b[i];
                  }
                  store8(out + gc, v);
                }
              }
            }
          }
        } else if (EPI == EPI_SWIGLU) {
          const long long ro = static_cast<long long>(row) * args.ld_out;
          const long long grow = args.drop.row0_global + row;
  #pragma unroll 1
          for (int c = 0; c < TILE_N / 32; ++c) {
            const int col = n0 + c * 32;
            if (col >= args.N) break;
            uint32_t rg[32], ru[32];
            tmem_ld_32x32(taddr + c * 32, rg);
            tmem_ld_32x32(taddr + TILE_N + c * 32, ru);
            tmem_ld_wait();
            if (row_ok) {
  #pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int gc = col + j * 8;
                if (gc < args.N) {
                  float g[8], u[8], h[8];
  #pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    g[i] = __uint_as_float(rg[j * 8 + i]);
                    u[i] = __uint_as_float(ru[j * 8 + i]);
                  }
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
                  if (out1) {  // keep the pre-activations for the backward pass
                    store8(out1 + ro + gc, g);
                    store8(out2 + ro + gc, u);
                  }
  #pragma unroll
                  for (int i = 0; i < 8; ++i) h[i] = g[i] * sigmoid_f(g[i]) * u[i];
                  if (drop_on) {
                    float f[8];
                    dropout_factors8(args.drop, grow, args.drop.col0_global + gc, f);
  #pragma unroll
                    for (int i = 0; i < 8; ++i) h[i] *= f[i];
                  }
                  store8(out0 + ro + gc, h);
                }
              }
            }
          }
        } else {  // EPI_DHIDDEN
          const long long ro = static_cast<long long>(row) * args.ld_out;
          const long long ri = static_cast<long long>(row) * args.ld_in;
          const long long grow = args.drop.row0_global + row;
  #pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int col = n0 + c * 32;
            if (col >= args.N) break;
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
            if (row_ok) {
  #pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int gc = col + j * 8;
                if (gc < args.N) {
                  float dh[8], g[8], u[8], dg[8], du[8];
  #pragma unroll
                  for (int i = 0; i < 8; ++i) dh[i] = __uint_as_float(r[j * 8 + i]);
                  load8(in0 + ri + gc, g);
                  load8(in1 + ri + gc, u);
                  if (drop_on) {
                    float f[8];
                    dropout_factors8(args.drop, grow, args.drop.col0_global + gc, f);
  #pragma unroll
                    for (int i = 0; i < 8; ++i) dh[i] *= f[i];
                  }
  #pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float s = sigmoid_f(g[i]);
                    du[i] = dh[i] * g[i] * s;
                    dg[i] = dh[i] * u[i] * s * (1.0f + g[i] * (1.0f - s));
                  }
                  store8(out0 + ro + gc, dg);
                  store8(out1 + ro + gc, du);
                }
              }
            }
          }
        }
}

// ------------------------------------------------------------------ kernel --
template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA0,
                    const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, const GemmArgs args) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "tcgen05 N range for M = 128");
  static_assert(!(EPI == EPI_SWIGLU) || (BN == 256 && !B_MN), "gate|up tile is 128 + 128 rows");
  static_assert(!B_MN || BN % 64 == 0, "MN-major B arrives in 64-column boxes");
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
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;

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
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
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
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
            ok = false;
            break;
          }
          const int seg = kb >= args.kb0 ? 1 : 0;
          const int k0 = (seg ? kb - args.kb0 : kb) * BK;
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
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    T* const out0 = static_cast<T*>(args.out0);
    T* const out1 = static_cast<T*>(args.out1);
    T* const out2 = static_cast<T*>(args.out2);
    const T* const in0 = static_cast<const T*>(args.in0);
    const T* const in1 = static_cast<const T*>(args.in1);
    const T* const bias0 = static_cast<const T*>(args.bias0);
    const T* const bias1 = static_cast<const T*>(args.bias1);
    const bool drop_on = args.drop.thresh != 0u;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(tfull_bar(acc), acc_phase, abortp);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + lane_addr;
      const int row = tc.m_tile * BM + row_in_tile;
      const int n0 = tc.n_tile * TILE_N;

      epilogue_tile<BN, EPI, T>(args, taddr, row, tc.batch, n0, out0, out1, out2, in0, in1, bias0, bias1,
                                drop_on);
      // The accumulator has been read: hand it back to the MMA issuer.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
    }
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
//   tempty[a]  lives in the leader, 8 arrivals: 4 epilogue warps of each CTA.
template <int BN, int STAGES>
constexpr size_t gemm_pair_smem_bytes() {
  return static_cast<size_t>(STAGES) * (BM * 128 + (BN / 2) * 128) + 1024;
}

template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA0,
                         const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmB0,
                         const __grid_constant__ CUtensorMap tmB1, const GemmArgs args) {
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tcgen05 N range for M = 256");
  static_assert(!(EPI == EPI_SWIGLU) || (BN == 256 && !B_MN), "gate|up tile is 128 + 128 rows");
  static_assert(!B_MN || BN % 128 == 0, "MN-major B arrives in 64-column boxes per CTA");
  constexpr int HALF_N = BN / 2;  // B columns staged by each CTA
  constexpr uint32_t A_BYTES = BM * 128;
  constexpr uint32_t B_BYTES = HALF_N * 128;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = tmem_cols_for(BN);
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  constexpr int PAIR_M = 2 * BM;
  constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, B_LBO = B_MN ? BK * 128 : 16;
  constexpr uint32_t A_KSTEP = (A_MN ? 2048 : 32) >> 4, B_KSTEP = (B_MN ? 2048 : 32) >> 4;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;

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
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps in each CTA of the pair
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
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
            ok = false;
            break;
          }
          const int seg = kb >= args.kb0 ? 1 : 0;
          const int k0 = (seg ? kb - args.kb0 : kb) * BK;
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
            for (int j = 0; j < HALF_N / 64; ++j)
              tma_load_2d_pair(sb + j * (BK * 128), mb, fb,
                               n0 + static_cast<int>(rank) * HALF_N + 64 * j, k0);
          } else {
            tma_load_2d_pair(sb, mb, fb, k0, n0 + static_cast<int>(rank) * HALF_N);
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
            umma_f16_pair(d_tmem, adesc + static_cast<uint64_t>(k * A_KSTEP),
                          bdesc + static_cast<uint64_t>(k * B_KSTEP), args.idesc,
                          (kb | k) != 0 ? 1u : 0u);
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
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    T* const out0 = static_cast<T*>(args.out0);
    T* const out1 = static_cast<T*>(args.out1);
    T* const out2 = static_cast<T*>(args.out2);
    const T* const in0 = static_cast<const T*>(args.in0);
    const T* const in1 = static_cast<const T*>(args.in1);
    const T* const bias0 = static_cast<const T*>(args.bias0);
    const T* const bias1 = static_cast<const T*>(args.bias1);
    const bool drop_on = args.drop.thresh != 0u;
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles; tile += num_pairs, ++local) {
      const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(tfull_bar(acc), acc_phase, abortp);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + lane_addr;
      const int row = tc.m_tile * PAIR_M + static_cast<int>(rank) * BM + row_in_tile;
      const int n0 = tc.n_tile * TILE_N;
      epilogue_tile<BN, EPI, T>(args, taddr, row, tc.batch, n0, out0, out1, out2, in0, in1, bias0,
                                bias1, drop_on);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
    }
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
