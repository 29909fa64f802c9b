// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused gated-MLP
// epilogues. One CTA per SM walks a grouped tile order; per CTA:
//   warp 0 (one lane)  TMA producer: fills a STAGES-deep shared-memory ring
//   warp 1 (one lane)  MMA issuer: tcgen05.mma into one of two TMEM accumulators
//   warps 2..17        epilogue: tcgen05.ld the finished accumulator, apply the
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
  EPI_STORE_TMA = 3,  // EPI_STORE through staged TMA stores (short reductions, see below)
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
constexpr int GEMM_THREADS = 576;  // producer warp, MMA warp, 16 epilogue warps

__host__ __device__ constexpr uint32_t tmem_cols_for(int bn) {
  return (2 * bn <= 32) ? 32u : (2 * bn <= 64) ? 64u : (2 * bn <= 128) ? 128u
         : (2 * bn <= 256) ? 256u : 512u;
}

// Epilogue warps and their staging buffers (see epilogue_tile below). The four warps
// that share a column part (one per TMEM lane quarter) form a GROUP: together they
// own all 128 rows of a 16-column unit, stage it as one [128 x 16] block (4 KB) and
// one of them issues one TMA operation for it.
constexpr int EPI_WARPS = 16;
constexpr int EPI_PARTS = EPI_WARPS / 4;                  // groups
constexpr int STAGE_BUF_BYTES = 128 * 32;                 // 128 rows x 16 sixteen-bit values
constexpr int STAGE_RING = 4;                             // buffers per group
constexpr int STAGING_BYTES = EPI_PARTS * STAGE_RING * STAGE_BUF_BYTES;  // 64 KB

// Operand ring + (for the staged epilogues) the store staging area + alignment slack.
template <int BN, int STAGES, int EPI>
constexpr size_t gemm_smem_bytes() {
  return static_cast<size_t>(STAGES) * (BM * 128 + BN * 128) + (EPI == EPI_STORE ? 0 : (EPI == EPI_DHIDDEN ? 96 * 1024 : STAGING_BYTES)) + 1024;
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

// sigma(x) = 1 / (1 + e^-x) = 0.5 * tanh(x / 2) + 0.5: one MUFU op and two FMAs. The
// hardware tanh approximation has a maximum relative error of about 2^-11, far below
// the resolution of the 16-bit outputs.
__device__ __forceinline__ float sigmoid_f(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
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

// Epilogue warps: EPI_WARPS = 16, four per TMEM lane quarter. Warp e (0..15) reads
// lanes 32 * (e & 3) and column part (e >> 2) of the tile.
//
// Output path. A thread owns one output ROW, so writing its values straight to global
// memory makes every store instruction touch 32 different cache lines with 16 bytes
// each; measured on the training shape, each extra output matrix written that way cost
// as much as a third of the whole GEMM. Instead the four warps of a group stage a
// [128 rows x 16 columns] block (4 KB, 32-byte rows, 32-byte swizzle) in shared memory
// and one thread hands it to the TMA store engine, which writes full 32-byte sectors,
// clips rows >= M and columns >= N by itself and runs asynchronously. Blocks are this
// large because the TMA engine of an SM retires roughly one operation per 90 cycles:
// with one [32 x 16] block per warp the dH epilogue alone needed 256 operations per
// tile and ran at exactly that rate.
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

__device__ __forceinline__ void group_sync(int gid) {
  asm volatile("bar.sync %0, 128;" ::"r"(gid) : "memory");  // the four warps of one group
}

// A group's ring of staging buffers and the bookkeeping for its TMA stores. Every
// member of the group holds a copy and calls the same sequence of methods.
struct StoreRing {
  uint32_t base;     // shared::cta address of this group's STAGE_RING buffers
  uint32_t row_off;  // byte offset of this thread's row inside a block
  uint32_t sw;       // 32-byte swizzle of that row: 16 when its two halves swap places
  int next;          // buffer the next block goes to
  int gid;           // named barrier of the group
  bool issuer;       // the one thread of the group that talks to the TMA engine

  __device__ __forceinline__ uint32_t current() const { return base + next * STAGE_BUF_BYTES; }
  // This thread's 16 values (two 16-byte halves) of its row. In the swizzled layout the
  // halves swap places in rows 4..7 of every group of 8, which spreads a warp's 16-byte
  // accesses over all banks.
  __device__ __forceinline__ void write(uint32_t buf, const uint4& lo, const uint4& hi) const {
    st_shared_v4(buf + row_off + sw, lo);
    st_shared_v4(buf + row_off + (16u ^ sw), hi);
  }
  // Hand the filled buffer to the TMA engine: block origin (col, row0) in the output.
  // Before the group barrier the issuer makes sure the buffer that comes NEXT is no
  // longer being read (it was used STAGE_RING - 1 flushes ago), so after the barrier
  // every member may start filling it.
  __device__ __forceinline__ void flush(uint32_t buf, const CUtensorMap* map, int col, int row0) {
    fence_proxy_async_smem();  // generic-proxy writes above -> visible to the async proxy
    if (issuer) tma_store_wait_read<STAGE_RING - 2>();
    group_sync(gid);
    if (issuer) {
      tma_store_2d(map, buf, col, row0);
      tma_store_commit();
    }
    next = (next + 1) % STAGE_RING;
  }
  __device__ __forceinline__ void drain() const {
    if (issuer) tma_store_wait_all();
  }
};

// Epilogue of one 128-row accumulator tile, executed by one warp for its 32 TMEM
// lanes and its part of the tile's columns: lane i owns output row
// tile_row0 + 32 * quarter + i and walks the columns in units of 16. `taddr` addresses
// (lane quarter, first accumulator column of the tile). All four warps of a group
// execute the same sequence of ring flushes (the conditions around them depend on
// columns only, never on the warp's rows).
template <int BN, int EPI, typename T>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& args, uint32_t taddr, int tile_row0,
                                              int quarter, int lane, int batch, int n0, int part,
                                              StoreRing& ring, const CUtensorMap* mo0,
                                              const CUtensorMap* mo1, const CUtensorMap* mo2,
                                              const T* in0, const T* in1, const T* bias0,
                                              const T* bias1, bool drop_on) {
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  constexpr int NU = TILE_N / 16 / EPI_PARTS;  // 16-column units per warp
  static_assert(NU >= 1, "tile too narrow for the column parts");
  const int row = tile_row0 + quarter * 32 + lane;
  const bool row_ok = row < args.M;
  const int u0 = part * NU;

  if (EPI == EPI_STORE) {
    // One output matrix behind a long main loop: direct 16-byte stores keep up (the
    // tensor pipe stays above 95 % busy), so this path spends no shared memory on
    // staging and keeps a deeper operand ring instead.
    T* const out = static_cast<T*>(batch ? args.out1 : args.out0) + static_cast<long long>(row) * args.ld_out;
    const T* const res = in0 ? in0 + static_cast<long long>(row) * args.ld_in : nullptr;
#pragma unroll
    for (int ui = 0; ui < NU; ++ui) {
      const int col = n0 + (u0 + ui) * 16;
      uint32_t acc[16];
      tmem_ld_32x16(taddr + (u0 + ui) * 16, acc);
      tmem_ld_wait();
      if (row_ok && col < args.N) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int gc = col + j * 8;
          if (gc < args.N) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[j * 8 + i]);
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
  } else if (EPI == EPI_STORE_TMA) {
    // Same result as EPI_STORE. When the reduction is short the main loop of a tile is
    // too brief to hide row-wise global stores, so the block goes out through the
    // staging ring and the TMA store engine instead (at the price of one ring stage).
    const CUtensorMap* mo = batch ? mo1 : mo0;
    const T* const res = in0 ? in0 + static_cast<long long>(row) * args.ld_in : nullptr;
#pragma unroll
    for (int ui = 0; ui < NU; ++ui) {
      const int col = n0 + (u0 + ui) * 16;
      uint32_t acc[16];
      tmem_ld_32x16(taddr + (u0 + ui) * 16, acc);
      tmem_ld_wait();
      if (col < args.N) {  // uniform over the group
        uint4 q[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int gc = col + j * 8;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[j * 8 + i]);
          if (gc < args.N) {
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
          q[j] = pack8<T>(v);
        }
        const uint32_t buf = ring.current();
        ring.write(buf, q[0], q[1]);
        ring.flush(buf, mo, col, tile_row0);
      }
    }
  } else if (EPI == EPI_SWIGLU) {
    const long long grow = args.drop.row0_global + row;
#pragma unroll
    for (int ui = 0; ui < NU; ++ui) {
      const int col = n0 + (u0 + ui) * 16;
      uint32_t rg[16], ru[16];
      tmem_ld_32x16(taddr + (u0 + ui) * 16, rg);
      tmem_ld_32x16(taddr + TILE_N + (u0 + ui) * 16, ru);
      tmem_ld_wait();
      if (col < args.N) {  // uniform over the group
        uint4 qh[2], qg[2], qu[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int gc = col + j * 8;
          float g[8], u[8], h[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            g[i] = __uint_as_float(rg[j * 8 + i]);
            u[i] = __uint_as_float(ru[j * 8 + i]);
          }
          if (gc < args.N) {
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
          if (mo1) {  // keep the pre-activations for the backward pass
            qg[j] = pack8<T>(g);
            qu[j] = pack8<T>(u);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] = g[i] * sigmoid_f(g[i]) * u[i];
          if (drop_on) {
            float f[8];
            dropout_factors8(args.drop, grow, args.drop.col0_global + gc, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] *= f[i];
          }
          qh[j] = pack8<T>(h);
        }
        uint32_t buf = ring.current();
        ring.write(buf, qh[0], qh[1]);
        ring.flush(buf, mo0, col, tile_row0);
        if (mo1) {
          buf = ring.current();
          ring.write(buf, qg[0], qg[1]);
          ring.flush(buf, mo1, col, tile_row0);
          buf = ring.current();
          ring.write(buf, qu[0], qu[1]);
          ring.flush(buf, mo2, col, tile_row0);
        }
      }
    }
  }
}

// --------------------------------------------------------- dH epilogue (B1) ----
// The dH epilogue needs G and U at the accumulator's positions. Reading them row by
// row from global memory has the same problem as writing row by row, so each group
// brings them in with TMA as [128 x 16] blocks, one 8 KB (G, U) buffer pair per
// 16-column unit, computes dGate / dUp in place (each thread overwrites exactly the 32
// bytes of G and of U it has just read) and hands the same buffers to the TMA store
// engine. Three pairs per group: the loads of unit k+1 are in flight while unit k is
// computed and while the stores of unit k-1 drain. The prefetch runs across tile
// boundaries, since G and U do not depend on the GEMM.
constexpr int DH_PAIRS = 3;
constexpr int DH_PAIR_BYTES = 2 * STAGE_BUF_BYTES;
constexpr int DH_STAGING_BYTES = EPI_PARTS * DH_PAIRS * DH_PAIR_BYTES;  // 96 KB
static_assert(DH_STAGING_BYTES == 96 * 1024, "keep gemm_smem_bytes in step");

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 q;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
               : "r"(addr)
               : "memory");
  return q;
}

// The epilogue role of one warp for all tiles of its CTA (or CTA pair).
//   TILE_M     rows per tile: 128, or 256 for a CTA pair (row_off = cluster rank * 128)
//   tfull0 / tempty0   shared::cta addresses of tfull[0] / tempty[0] ([1] is 8 bytes on)
//   REMOTE     tempty lives in the pair's leader CTA: arrive through the cluster
//   epi_smem   this CTA's epilogue staging area; lbar0: DH_PAIRS load barriers per group
//   grp_abort  one word per group, written by the group's issuer warp only
//
// Staged epilogues synchronise the four warps of a group with named barriers, which
// have no time limit. To keep every wait in the kernel bounded, only the group's issuer
// warp (lane quarter 0) waits on mbarriers; it publishes the outcome in grp_abort before
// the next group barrier and all four warps act on that one word, so they always take
// the same way out.
template <int BN, int EPI, typename T, int TILE_M, bool REMOTE>
__device__ __forceinline__ void epilogue_role(
    const GemmArgs& args, int warp, int lane, int first_tile, int tile_stride, int total_tiles,
    int m_tiles, int n_tiles, int row_off, uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
    uint32_t epi_smem, uint32_t lbar0, int* grp_abort_all, const CUtensorMap* mo0,
    const CUtensorMap* mo1_in, const CUtensorMap* mo2, const CUtensorMap* mi0,
    const CUtensorMap* mi1, int* abort_flag) {
  constexpr int TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  constexpr bool GROUPED = (EPI != EPI_STORE);
  volatile int* abortp = abort_flag;
  const int ew = warp - 2;          // epilogue warp index 0..15
  const int quarter = warp & 3;     // TMEM lanes this warp may read
  const int col_part = ew >> 2;
  const int gid = 1 + col_part;     // named barrier of this warp's group
  const bool issuer_warp = quarter == 0;
  const bool issuer = issuer_warp && lane == 0;
  volatile int* grp_abort = grp_abort_all + col_part;
  const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
  const uint32_t row_off_bytes = static_cast<uint32_t>(quarter * 32 + lane) * 32u;
  const uint32_t sw = static_cast<uint32_t>((lane >> 2) & 1) << 4;
  const T* const in0 = static_cast<const T*>(args.in0);
  const T* const in1 = static_cast<const T*>(args.in1);
  const T* const bias0 = static_cast<const T*>(args.bias0);
  const T* const bias1 = static_cast<const T*>(args.bias1);
  const CUtensorMap* const mo1 = (EPI == EPI_STORE_TMA || args.out1) ? mo1_in : nullptr;
  const bool drop_on = args.drop.thresh != 0u;
  bool ok = true;
  int local = 0;

  auto release_tmem = [&](int acc) {
    // Every tcgen05.ld of this tile was followed by tcgen05.wait::ld, so the data is in
    // registers: hand the TMEM buffer back to the MMA issuer. The arrive has release
    // semantics; no fence is placed here on purpose, since a fence would also wait for
    // this warp's outstanding global stores.
    __syncwarp();
    if (lane == 0) {
      if (REMOTE) mbar_arrive_cluster(mapa_shared(tempty0 + 8u * acc, 0));
      else mbar_arrive(tempty0 + 8u * acc);
    }
  };
  // Wait for the accumulator of the warp's `local`-th tile; false = give up.
  auto wait_tile = [&](int acc) -> bool {
    if (!GROUPED) {
      bool w = mbar_wait(tfull0 + 8u * acc, (local >> 1) & 1, abortp);
      return __all_sync(0xffffffffu, w);
    }
    if (issuer_warp) {
      bool w = mbar_wait(tfull0 + 8u * acc, (local >> 1) & 1, abortp);
      w = __all_sync(0xffffffffu, w);
      if (lane == 0) *grp_abort = (!w || *abortp != 0) ? 1 : 0;
    }
    group_sync(gid);
    const bool go = *grp_abort == 0;
    group_sync(gid);  // nobody reads the word after this point until it is written again
    return go;
  };

  if (EPI != EPI_DHIDDEN) {
    StoreRing ring{epi_smem + col_part * (STAGE_RING * STAGE_BUF_BYTES), row_off_bytes, sw, 0, gid, issuer};
    for (int tile = first_tile; tile < total_tiles; tile += tile_stride, ++local) {
      const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
      const int acc = local & 1;
      ok = wait_tile(acc);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + lane_addr;
      epilogue_tile<BN, EPI, T>(args, taddr, tc.m_tile * TILE_M + row_off, quarter, lane, tc.batch,
                                tc.n_tile * TILE_N, col_part, ring, mo0, mo1, mo2, in0, in1, bias0,
                                bias1, drop_on);
      release_tmem(acc);
    }
    if (GROUPED) ring.drain();  // shared memory must stay valid until TMA has read it
  } else {
    constexpr int NU = BN / 16 / EPI_PARTS;  // 16-column units per group and tile
    const uint32_t grp_smem = epi_smem + col_part * (DH_PAIRS * DH_PAIR_BYTES);
    const uint32_t grp_bar = lbar0 + 8u * (col_part * DH_PAIRS);
    // Origin (first row of this CTA's 128-row slab, first column of this group's part) of
    // `tile`: decoded once per tile, never per unit (decode_tile divides by run-time values).
    auto tile_origin = [&](int tile, int& row0, int& col0) {
      const TileCoord tc = decode_tile(tile, m_tiles, n_tiles, args.group_m);
      row0 = tc.m_tile * TILE_M + row_off;
      col0 = tc.n_tile * TILE_N + col_part * NU * 16;
    };
    // Issue the G / U loads of unit number k, block origin (col, row0) (issuer only).
    auto issue_load = [&](int k, int row0, int col) {
      const int p = k % DH_PAIRS;
      // This runs before the stores of unit k-1 are issued. The pair was last read by the
      // two stores of unit k-3; the only groups committed since are the two of unit k-2.
      tma_store_wait_read<2>();
      const uint32_t buf = grp_smem + p * DH_PAIR_BYTES;
      const uint32_t bar = grp_bar + 8u * p;
      mbar_expect_tx(bar, DH_PAIR_BYTES);
      tma_load_2d(buf, mi0, bar, col, row0);
      tma_load_2d(buf + STAGE_BUF_BYTES, mi1, bar, col, row0);
    };
    int k = 0;
    int row0 = 0, col0 = 0, next_row0 = 0, next_col0 = 0;
    if (first_tile < total_tiles) {
      tile_origin(first_tile, row0, col0);
      if (issuer) issue_load(0, row0, col0);
    }
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_stride, ++local) {
      const bool has_next = tile + tile_stride < total_tiles;
      if (has_next) tile_origin(tile + tile_stride, next_row0, next_col0);
      const int acc = local & 1;
      ok = wait_tile(acc);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + lane_addr + col_part * NU * 16;
      const long long grow = args.drop.row0_global + row0 + quarter * 32 + lane;
#pragma unroll 1
      for (int ui = 0; ui < NU; ++ui, ++k) {
        // prefetch the next unit's G and U (possibly the first unit of the next tile)
        if (issuer) {
          if (ui + 1 < NU) issue_load(k + 1, row0, col0 + (ui + 1) * 16);
          else if (has_next) issue_load(k + 1, next_row0, next_col0);
        }
        const int col = col0 + ui * 16;
        uint32_t acc_r[16];
        tmem_ld_32x16(taddr + ui * 16, acc_r);
        const int p = k % DH_PAIRS;
        if (issuer_warp) {
          bool w = mbar_wait(grp_bar + 8u * p, (k / DH_PAIRS) & 1, abortp);
          w = __all_sync(0xffffffffu, w);
          if (lane == 0) *grp_abort = (!w || *abortp != 0) ? 1 : 0;
        }
        group_sync(gid);  // G and U of this unit have landed (or the group gives up)
        tmem_ld_wait();
        if (*grp_abort != 0) {
          ok = false;
          break;
        }
        const uint32_t gbuf = grp_smem + p * DH_PAIR_BYTES + row_off_bytes;
        const uint32_t ubuf = gbuf + STAGE_BUF_BYTES;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float dh[8], g[8], u[8], dg[8], du[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) dh[i] = __uint_as_float(acc_r[j * 8 + i]);
          unpack8<T>(ld_shared_v4(gbuf + ((j * 16) ^ sw)), g);
          unpack8<T>(ld_shared_v4(ubuf + ((j * 16) ^ sw)), u);
          if (drop_on) {
            float f[8];
            dropout_factors8(args.drop, grow, args.drop.col0_global + col + j * 8, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) dh[i] *= f[i];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float sg = sigmoid_f(g[i]);
            du[i] = dh[i] * g[i] * sg;
            dg[i] = dh[i] * u[i] * sg * (1.0f + g[i] * (1.0f - sg));
          }
          st_shared_v4(gbuf + ((j * 16) ^ sw), pack8<T>(dg));
          st_shared_v4(ubuf + ((j * 16) ^ sw), pack8<T>(du));
        }
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA store
        group_sync(gid);
        if (issuer) {
          // Rows >= M and columns >= N of a block are clipped by the hardware.
          tma_store_2d(mo0, grp_smem + p * DH_PAIR_BYTES, col, row0);
          tma_store_commit();
          tma_store_2d(mo1_in, grp_smem + p * DH_PAIR_BYTES + STAGE_BUF_BYTES, col, row0);
          tma_store_commit();
        }
      }
      if (!ok) break;
      release_tmem(acc);
      row0 = next_row0;
      col0 = next_col0;
    }
    if (issuer) tma_store_wait_all();
  }
  if (!ok && lane == 0) {
    *abort_flag = 1;
    atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
  }
}

// ------------------------------------------------------------------ kernel --
template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA0,
                    const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CUtensorMap tmO0,
                    const __grid_constant__ CUtensorMap tmO1,
                    const __grid_constant__ CUtensorMap tmO2,
                    const __grid_constant__ CUtensorMap tmI0,
                    const __grid_constant__ CUtensorMap tmI1, const GemmArgs args) {
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
  // dH epilogue only: one barrier per (epilogue group, G/U buffer pair)
  __shared__ __align__(8) uint64_t lbars[EPI == EPI_DHIDDEN ? EPI_PARTS * DH_PAIRS : 1];
  __shared__ int grp_abort[EPI_PARTS];

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
    for (int i = 0; i < EPI_PARTS; ++i) grp_abort[i] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EPI_WARPS);  // one arrival per epilogue warp
    }
    if (EPI == EPI_DHIDDEN)
      for (int i = 0; i < EPI_PARTS * DH_PAIRS; ++i) mbar_init(smem_u32(lbars) + 8u * i, 1);
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
    epilogue_role<BN, EPI, T, BM, false>(args, warp, lane, blockIdx.x, gridDim.x, total_tiles, m_tiles,
                                         n_tiles, 0, tmem_base, tfull_bar(0), tempty_bar(0),
                                         smem_base + STAGES * STAGE_BYTES, smem_u32(lbars), grp_abort, &tmO0,
                                         &tmO1, &tmO2, &tmI0, &tmI1, &abort_flag);
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
template <int BN, int STAGES, int EPI>
constexpr size_t gemm_pair_smem_bytes() {
  return static_cast<size_t>(STAGES) * (BM * 128 + (BN / 2) * 128) + (EPI == EPI_STORE ? 0 : (EPI == EPI_DHIDDEN ? 96 * 1024 : STAGING_BYTES)) + 1024;
}

template <int BN, bool A_MN, bool B_MN, int EPI, typename T, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA0,
                         const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmB0,
                         const __grid_constant__ CUtensorMap tmB1,
                         const __grid_constant__ CUtensorMap tmO0,
                         const __grid_constant__ CUtensorMap tmO1,
                         const __grid_constant__ CUtensorMap tmO2,
                    const __grid_constant__ CUtensorMap tmI0,
                    const __grid_constant__ CUtensorMap tmI1, const GemmArgs args) {
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
  // dH epilogue only: one barrier per (epilogue group, G/U buffer pair)
  __shared__ __align__(8) uint64_t lbars[EPI == EPI_DHIDDEN ? EPI_PARTS * DH_PAIRS : 1];
  __shared__ int grp_abort[EPI_PARTS];

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
    for (int i = 0; i < EPI_PARTS; ++i) grp_abort[i] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * EPI_WARPS);  // the epilogue warps of both CTAs of the pair
    }
    if (EPI == EPI_DHIDDEN)
      for (int i = 0; i < EPI_PARTS * DH_PAIRS; ++i) mbar_init(smem_u32(lbars) + 8u * i, 1);
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
    epilogue_role<BN, EPI, T, PAIR_M, true>(args, warp, lane, pair, num_pairs, total_tiles, m_tiles,
                                            n_tiles, static_cast<int>(rank) * BM, tmem_base, tfull_bar(0),
                                            tempty_bar(0), smem_base + STAGES * STAGE_BYTES,
                                            smem_u32(lbars), grp_abort, &tmO0, &tmO1, &tmO2, &tmI0,
                                            &tmI1, &abort_flag);
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
