// Skinny-M (decode) forward: M <= 64 tokens, so the cost is one pass over the
// weights and the kernels are bound by HBM bandwidth, not by tensor throughput.
//
// Layout of the work ("swap-AB"): the 128 TMEM lanes / MMA rows are 128 WEIGHT rows
// and the (padded) token count MPAD in {16, 32, 64} is the MMA N dimension, so a
// 16 KB weight tile [128 x 64] is used once by one small tcgen05.mma group and
// the tensor pipe stays far below its limit while TMA streams the weights.
//
// Balance ("stream-K"): the work is the list of (weight row tile, 64-wide
// reduction block) units in row-tile-major order. CTA c of G takes the
// contiguous unit range [c*U/G, (c+1)*U/G): every CTA streams the same number of
// weight bytes (to within one unit) whatever the tile count is. A row tile whose
// reduction is split across CTAs is finished by its owner, the contributor that holds
// the tile's first reduction blocks: every other contributor stores its fp32 partial
// tile to its scratch slot and adds its block count to the tile's counter; the owner,
// for which the tile is the last thing it works on, waits (bounded) until the others'
// blocks are all counted, adds their partials to its own accumulators in CTA order (so
// the result does not depend on arrival order), applies the epilogue and clears the
// counter. With two contributors per tile, the usual case, the other part was
// published a whole kernel earlier and the owner never actually waits. Only owners
// wait, and only after they have published everything they owe, so no CTA waits for one
// that is itself waiting; the grid is at most one CTA per SM, so a contributor that has
// not started yet is only waiting for an SM that some other kernel still holds, and the
// wait gives up (status word, no output for that tile) after WAIT_LIMIT_CYCLES.
//
//   DUAL = true   H^T[n, m]  = silu(Wg[n,:].x[m,:] + bg[n]) * (Wu[n,:].x[m,:] + bu[n])
//                 two accumulators (gate, up) per tile, written as H[m, n]
//   DUAL = false  Y^T[k, m]  = Wd[k,:].h[m,:] + bd[k], written as Y[m, k]
#pragma once
#include "gemm_tcgen05.cuh"

namespace gmlp {

struct DecodeArgs {
  int M;          // tokens (<= MPAD)
  int rows;       // weight rows: N for DUAL, K (hidden) otherwise
  int kbt;        // 64-wide reduction blocks per row tile
  uint32_t idesc;
  int* status;
  const void* bias0;  // per weight row (gate bias, or down bias)
  const void* bias1;  // up bias (DUAL)
  void* out;          // H[M, rows] or Y[M, rows]
  const void* residual;  // optional [M, rows] added to the output (down projection only)
  const float* row_scale;  // optional [M] per-token factors on the accumulators before the bias
  const float* wscale0;    // optional [rows] per-weight-row factors (8-bit weights: their dequantisation scales)
  const float* wscale1;    // the same for the second weight matrix (DUAL)
  long long ld_out;
  float* slots;       // [2 * gridDim.x][NACC][128][MPAD] fp32 partial tiles
  int* counters;      // [row tiles] reduction blocks whose partials are in the slots; zero on entry, and on exit
                      // unless the kernel gave up a wait (status word != 0): then the host clears them
  int act;            // gate activation (ACT_*), DUAL only
  int dependent;      // 1: launched with programmatic stream serialization behind the kernel
                      //    that produces the activations (and last used slots / counters)
};

// Programmatic dependent launch. launch_dependents lets the next kernel in the stream
// start filling SMs as this grid's CTAs retire; wait blocks until the preceding grid has
// completed and its memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

constexpr int DECODE_THREADS = 192;
// One CTA per SM, one weight sub-tile per unit (two CTAs per SM with half the ring each,
// and larger units with whole row tiles owned by CTAs, were both slower).
#ifndef GMLP_DECODE_SUB64_DUAL
#define GMLP_DECODE_SUB64_DUAL 1
#endif
#ifndef GMLP_DECODE_SUB64_DOWN
#define GMLP_DECODE_SUB64_DOWN 1
#endif
#ifndef GMLP_DECODE_SUB32_DUAL
#define GMLP_DECODE_SUB32_DUAL 1
#endif
#ifndef GMLP_DECODE_SUB32_DOWN
#define GMLP_DECODE_SUB32_DOWN 1
#endif
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_subtiles() {
  return MPAD == 64 ? (DUAL ? GMLP_DECODE_SUB64_DUAL : GMLP_DECODE_SUB64_DOWN)
         : MPAD == 32 ? (DUAL ? GMLP_DECODE_SUB32_DUAL : GMLP_DECODE_SUB32_DOWN) : 1;
}
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_stage_bytes() {
  return (DUAL ? 2 : 1) * decode_subtiles<MPAD, DUAL>() * 16384 + MPAD * 128;
}
// As many stages as fit in shared memory: bytes in flight per SM are what hides the
// DRAM latency.
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_stages() {
  constexpr int fit = (232448 - 1024 - 512) / decode_stage_bytes<MPAD, DUAL>();
  return fit > 12 ? 12 : fit;
}
template <int MPAD, bool DUAL>
constexpr size_t decode_smem_bytes() {
  return static_cast<size_t>(decode_stages<MPAD, DUAL>()) * decode_stage_bytes<MPAD, DUAL>() + 1024;
}
// Rows of one TMA box of weights: all sub-tiles of a matrix in one box when they fit
// the 256-row limit of a box, else in two.
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_box_rows() {
  return decode_subtiles<MPAD, DUAL>() >= 2 ? 256 : 128;
}

__device__ __forceinline__ long long unit_start(long long c, long long total, long long g) {
  return (c * total) / g;
}

// out[m * ld] = act(gate[m] + b0) * (up[m] + b1) for the tokens m < M of one weight row,
// with the activation a compile-time constant.
// With scales: gate and up are first multiplied by row_scale[m] (per token; null = 1) and by this
// weight row's own factors ws0 / ws1.
template <int ACT, int COUNT, typename T>
__device__ __forceinline__ void store_gated(T* po, long long ld, int M, const float* gate, const float* up,
                                            float b0, float b1, const float* row_scale, bool scaled, float ws0,
                                            float ws1) {
  if (!scaled) {
#pragma unroll
    for (int m = 0; m < COUNT; ++m)
      if (m < M) po[static_cast<long long>(m) * ld] = static_cast<T>(act_value(ACT, gate[m] + b0) * (up[m] + b1));
  } else {
#pragma unroll
    for (int m = 0; m < COUNT; ++m)
      if (m < M) {
        const float r = row_scale ? row_scale[m] : 1.0f;  // the same address for every lane: one broadcast load
        po[static_cast<long long>(m) * ld] =
            static_cast<T>(act_value(ACT, gate[m] * (r * ws0) + b0) * (up[m] * (r * ws1) + b1));
      }
  }
}

// FP8: weights and activations are e4m3 bytes (128 reduction elements per 128-byte row instead
// of 64), multiplied by tcgen05.mma.kind::f8f6f4; T is still the type of bias, residual and
// output. Everything else (rings, stream-K split, owners) is the same code.
template <int MPAD, bool DUAL, typename T, bool FP8 = false>
__global__ void __launch_bounds__(DECODE_THREADS, 1)
decode_stream_kernel(const __grid_constant__ CUtensorMap tmW0,
                     const __grid_constant__ CUtensorMap tmW1,
                     const __grid_constant__ CUtensorMap tmAct, const DecodeArgs args) {
  static_assert(MPAD == 16 || MPAD == 32 || MPAD == 64, "token padding");
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int SUB = decode_subtiles<MPAD, DUAL>();  // weight sub-tiles per unit
  constexpr int TILE_ROWS = 128 * SUB;                // weight rows per unit ("row tile")
  constexpr int BOX_ROWS = decode_box_rows<MPAD, DUAL>();
  constexpr int STAGES = decode_stages<MPAD, DUAL>();
  constexpr int RED = FP8 ? 128 : BK;      // reduction elements per stage: one 128-byte row
  constexpr uint32_t W_BYTES = 128 * 128;  // one [128 rows x 128 bytes] weight sub-tile
  constexpr uint32_t ACT_BYTES = MPAD * 128;
  constexpr uint32_t ACT_OFF = NACC * SUB * W_BYTES;  // stage: [W0 sub-tiles][W1 sub-tiles][activations]
  constexpr uint32_t STAGE_BYTES = ACT_OFF + ACT_BYTES;
  static_assert(STAGE_BYTES == decode_stage_bytes<MPAD, DUAL>(), "stage layout");
  constexpr uint32_t ACC_COLS = NACC * SUB * MPAD;  // TMEM columns per accumulator buffer
  constexpr uint32_t TMEM_COLS = (2 * ACC_COLS <= 32) ? 32 : (2 * ACC_COLS <= 64) ? 64
                                 : (2 * ACC_COLS <= 128) ? 128 : (2 * ACC_COLS <= 256) ? 256 : 512;
  static_assert(2 * ACC_COLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");

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
  const long long row_tiles = (args.rows + TILE_ROWS - 1) / TILE_ROWS;
  const long long total = row_tiles * args.kbt;
  const long long u_begin = unit_start(blockIdx.x, total, gridDim.x);
  const long long u_end = unit_start(blockIdx.x + 1, total, gridDim.x);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmW0);
    tma_prefetch_desc(&tmAct);
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
  if (threadIdx.x == 0) pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer --
    if (lane == 0) {
      // Weights are read exactly once: mark them evict-first so they do not push
      // the (re-used) activations out of L2.
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_a = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // (row tile, reduction block) of the unit being issued, kept incrementally: a 64-bit division per
      // unit costs the issuing thread a good part of the time one 16 KB unit takes to stream
      int w_tile = static_cast<int>(u_begin / args.kbt);
      int w_kb = static_cast<int>(u_begin - static_cast<long long>(w_tile) * args.kbt);
      int a_kb = w_kb;
      auto load_weights = [&](int st) {  // the next unit's weights
        const int tile = w_tile, kb = w_kb;
        if (++w_kb == args.kbt) {
          w_kb = 0;
          ++w_tile;
        }
        const uint32_t sw = smem_base + st * STAGE_BYTES;
        const uint32_t fb = full_bar(st);
        mbar_expect_tx(fb, STAGE_BYTES);
        // Rows past the end of the matrix (a last tile that is not full) arrive as zeros.
#pragma unroll
        for (int b = 0; b < TILE_ROWS / BOX_ROWS; ++b) {
          tma_load_2d_hint(sw + b * BOX_ROWS * 128, &tmW0, fb, kb * RED, tile * TILE_ROWS + b * BOX_ROWS, pol_w);
          if (DUAL)
            tma_load_2d_hint(sw + SUB * W_BYTES + b * BOX_ROWS * 128, &tmW1, fb, kb * RED,
                             tile * TILE_ROWS + b * BOX_ROWS, pol_w);
        }
      };
      auto load_act = [&](int st) {  // the next unit's activations (issued in the same order as the weights)
        const int kb = a_kb;
        if (++a_kb == args.kbt) a_kb = 0;
        tma_load_2d_hint(smem_base + st * STAGE_BYTES + ACT_OFF, &tmAct, full_bar(st), kb * RED, 0, pol_a);
      };
      long long u = u_begin;
      if (args.dependent) {
        // The weights do not depend on the preceding kernel: fill the ring with them while
        // that kernel's last CTAs are still running, then wait for it and add the
        // activations of the same stages.
        const long long n0 = (u_end - u_begin) < STAGES ? (u_end - u_begin) : STAGES;
        for (long long i = 0; i < n0; ++i) load_weights(static_cast<int>(i));
        pdl_wait();
        for (long long i = 0; i < n0; ++i) load_act(static_cast<int>(i));
        u = u_begin + n0;
        stage = static_cast<int>(n0 % STAGES);
        phase = (n0 == STAGES) ? 1u : 0u;
      }
      for (; u < u_end; ++u) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        load_weights(stage);
        load_act(stage);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
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
      int seg = 0;
      bool ok = true;
      long long u = u_begin;
      while (u < u_end && ok) {
        const long long tile = u / args.kbt;
        const long long tile_end = (tile + 1) * args.kbt;
        const long long seg_end = tile_end < u_end ? tile_end : u_end;
        const int acc = seg & 1;
        const uint32_t acc_phase = (seg >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        bool first = true;
        for (; u < seg_end; ++u) {
          if (!mbar_wait(full_bar(stage), phase, abortp)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_base + stage * STAGE_BYTES;
          const uint64_t xdesc = make_smem_desc(sw + ACT_OFF, 16, 1024);
#pragma unroll
          for (int t = 0; t < SUB; ++t) {
            const uint64_t w0desc = make_smem_desc(sw + t * W_BYTES, 16, 1024);
            const uint64_t w1desc = make_smem_desc(sw + (SUB + t) * W_BYTES, 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // four 32-byte steps per 128-byte row, whatever the element size
              const uint32_t accum = (first && k == 0) ? 0u : 1u;
              if (FP8) {
                umma_f8(d_tmem + (t * NACC) * MPAD, w0desc + static_cast<uint64_t>(2 * k),
                        xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
                if (DUAL)
                  umma_f8(d_tmem + (t * NACC + 1) * MPAD, w1desc + static_cast<uint64_t>(2 * k),
                          xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
              } else {
                umma_f16(d_tmem + (t * NACC) * MPAD, w0desc + static_cast<uint64_t>(2 * k),
                         xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
                if (DUAL)
                  umma_f16(d_tmem + (t * NACC + 1) * MPAD, w1desc + static_cast<uint64_t>(2 * k),
                           xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
              }
            }
          }
          first = false;
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(tfull_bar(acc));
        ++seg;
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;  // weight row inside the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int ep_tid = threadIdx.x - 64;  // 0..127 among the epilogue warps
    T* const out = static_cast<T*>(args.out);
    const T* const residual = static_cast<const T*>(args.residual);
    const T* const bias0 = static_cast<const T*>(args.bias0);
    const T* const bias1 = static_cast<const T*>(args.bias1);
    constexpr long long SUB_FLOATS = static_cast<long long>(NACC) * 128 * MPAD;  // one sub-tile's partial
    constexpr long long SLOT_FLOATS = SUB * SUB_FLOATS;
    if (args.dependent) pdl_wait();  // slots, counters and outputs may still be in use by the preceding grid
    int seg = 0;
    bool ok = true;
    long long u = u_begin;
    while (u < u_end) {
      const long long tile = u / args.kbt;
      const long long tile_begin = tile * args.kbt;
      const long long tile_end = tile_begin + args.kbt;
      const long long seg_end = tile_end < u_end ? tile_end : u_end;
      const bool complete = (u == tile_begin) && (seg_end == tile_end);
      const int acc = seg & 1;
      const uint32_t acc_phase = (seg >> 1) & 1;
      ok = mbar_wait_warp(tfull_bar(acc), acc_phase, abortp, lane);
      if (!ok && lane == 0) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
      }
      // The four epilogue warps meet at named barriers further down; they must all
      // take the same way out, so they VOTE on the outcome of the wait: the barrier
      // returns one answer to all 128 threads even if the abort flag (set at any time
      // by the producer or the MMA thread) flips between two warps' reads of it. Every
      // warp reaches this barrier because its wait above is bounded.
      if (named_bar_or(1, 128, *abortp != 0)) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + lane_addr;

      // All MPAD tokens of weight row `wrow`. The activation is chosen OUTSIDE the unrolled
      // token loop: with the switch inside, each of the 64 copies of the loop body carries
      // every activation's code and the taken path is 64 islands in 150 KB of instructions
      // run once per tile, which costs instruction fetch time at every tile.
      auto emit = [&](long long wrow, float b0, float b1, const float* first, const float* second) {
        if (wrow >= args.rows) return;
        T* const po = out + wrow;
        const bool scaled = args.row_scale != nullptr || args.wscale0 != nullptr;
        const float ws0 = args.wscale0 ? args.wscale0[wrow] : 1.0f;
        const float ws1 = (DUAL && args.wscale1) ? args.wscale1[wrow] : 1.0f;
        if (DUAL) {
          switch (args.act) {
            case ACT_SILU: store_gated<ACT_SILU, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
            case ACT_NONE: store_gated<ACT_NONE, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
            case ACT_RELU: store_gated<ACT_RELU, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
            case ACT_GELU: store_gated<ACT_GELU, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
            case ACT_SIGMOID:
              store_gated<ACT_SIGMOID, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled,
                                             ws0, ws1);
              break;
            case ACT_TANH: store_gated<ACT_TANH, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
            default: store_gated<ACT_LEAKY_RELU, MPAD>(po, args.ld_out, args.M, first, second, b0, b1, args.row_scale, scaled, ws0, ws1); break;
          }
        } else {
          const T* const pr = residual ? residual + wrow : nullptr;
#pragma unroll
          for (int m = 0; m < MPAD; ++m) {
            if (m < args.M) {
              float o = (scaled ? first[m] * ((args.row_scale ? args.row_scale[m] : 1.0f) * ws0) : first[m]) + b0;
              if (pr) o += static_cast<float>(pr[static_cast<long long>(m) * args.ld_out]);
              po[static_cast<long long>(m) * args.ld_out] = static_cast<T>(o);
            }
          }
        }
      };
      auto row_bias = [&](const T* bias, long long wrow) {
        return (bias && wrow < args.rows) ? static_cast<float>(bias[wrow]) : 0.f;
      };
      // A split row tile is finished by its OWNER, the contributor that holds the tile's
      // first reduction blocks: for that CTA the tile is the last thing it works on, while
      // for the contributor that holds the tile's last blocks it is the first, published
      // a whole kernel earlier. So the owner keeps its own part in registers, finds the
      // other parts (all of them, when a tile has two contributors) already counted,
      // fetches them in one round trip and adds them in CTA order, which makes the result
      // independent of arrival order. Everybody else stores its part, counts it and moves
      // on (or exits): nobody but an owner ever waits, and an owner has published
      // everything it owes before it does.
      const bool owner = !complete && (u == tile_begin);
      float4* const slot4 = reinterpret_cast<float4*>(args.slots + 2LL * blockIdx.x * SLOT_FLOATS);
      const long long c_first = ((tile_begin + 1) * gridDim.x - 1) / total;
      const long long c_last = (tile_end * gridDim.x - 1) / total;
      if (owner) {
        // the other contributors' reduction blocks must all be counted
        if (ep_tid == 0) {
          const int need = args.kbt - static_cast<int>(seg_end - u);
          const volatile int* cnt = args.counters + tile;
          const long long t0 = clock64();
          while (*cnt != need) {
            if (*abortp != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES) {
              abort_flag = 1;
              atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
              break;
            }
            __nanosleep(64);
          }
          __threadfence();
        }
        if (named_bar_or(1, 128, *abortp != 0)) break;
      }

#pragma unroll 1
      for (int t = 0; t < SUB; ++t) {
        float v[NACC][MPAD];
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
#pragma unroll
          for (int c = 0; c < MPAD / 16; ++c) {
            uint32_t r[16];
            tmem_ld_32x16(taddr + (t * NACC + a) * MPAD + c * 16, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[a][c * 16 + i] = __uint_as_float(r[i]);
          }
        }
        if (owner) {
          // The other parts, as many contributors per round trip as the operand ring holds:
          // cp.async copies them into the ring, which is idle (this is the CTA's last
          // segment and its MMAs have completed), each thread into a column of its own.
          constexpr int ITEM4 = NACC * (MPAD / 4);  // 16-byte pieces per contributor and thread
          constexpr int RING_CAP = static_cast<int>(STAGES * STAGE_BYTES / (128 * 16));
          constexpr int FIX_CONTRIB = RING_CAP / ITEM4;  // contributors fetched per round trip
          static_assert(ITEM4 <= RING_CAP, "the ring must hold one contributor's part");
          auto stage_addr = [&](int k) { return smem_base + static_cast<uint32_t>(k * 128 + ep_tid) * 16u; };
          for (long long cb = c_first + 1; cb <= c_last; cb += FIX_CONTRIB) {
            const long long ce = cb + FIX_CONTRIB - 1 < c_last ? cb + FIX_CONTRIB - 1 : c_last;
            int k = 0;
            for (long long c = cb; c <= ce; ++c) {
              const float4* s4 = reinterpret_cast<const float4*>(args.slots + 2LL * c * SLOT_FLOATS);
#pragma unroll
              for (int a = 0; a < NACC; ++a)
#pragma unroll
                for (int i = 0; i < MPAD / 4; ++i, ++k)
                  cp_async_16(stage_addr(k), s4 + ((t * NACC + a) * (MPAD / 4) + i) * 128 + r_in_tile);
            }
            cp_async_wait_all();
            k = 0;
            for (long long c = cb; c <= ce; ++c) {
#pragma unroll
              for (int a = 0; a < NACC; ++a)
#pragma unroll
                for (int i = 0; i < MPAD / 4; ++i, ++k) {
                  const float4 q = ld_shared_f4(stage_addr(k));
                  v[a][4 * i] += q.x;
                  v[a][4 * i + 1] += q.y;
                  v[a][4 * i + 2] += q.z;
                  v[a][4 * i + 3] += q.w;
                }
            }
          }
        }
        if (complete || owner) {
          const long long wrow = tile * TILE_ROWS + t * 128 + r_in_tile;
          emit(wrow, row_bias(bias0, wrow), DUAL ? row_bias(bias1, wrow) : 0.f, v[0], v[NACC - 1]);
        } else {
          // this CTA's part of the sub-tile goes to its slot. Slot layout: float4 (sub-tile t,
          // accumulator a, i, row) at index ((t * NACC + a) * MPAD/4 + i) * 128 + row, so that
          // the 32 lanes of a warp (32 consecutive rows) touch 512 contiguous bytes per access.
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int i = 0; i < MPAD / 4; ++i)
              slot4[((t * NACC + a) * (MPAD / 4) + i) * 128 + r_in_tile] =
                  make_float4(v[a][4 * i], v[a][4 * i + 1], v[a][4 * i + 2], v[a][4 * i + 3]);
        }
      }
      // TMEM has been read into registers: the MMA issuer may reuse the buffer.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));

      if (owner) {
        if (ep_tid == 0) args.counters[tile] = 0;  // leave the scratch ready for the next call
      } else if (!complete) {
        // count this CTA's reduction blocks once its part is visible
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (ep_tid == 0) atomicAdd(args.counters + tile, static_cast<int>(seg_end - u));
      }
      u = seg_end;
      ++seg;
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

}  // namespace gmlp
