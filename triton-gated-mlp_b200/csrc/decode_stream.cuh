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
// reduction is split across CTAs is finished by whichever contributor arrives
// last: each contributor stores its fp32 partial tile to its own scratch slot,
// bumps the tile's counter, and the one that completes the count sums all slots in
// CTA order (so the result does not depend on arrival order), applies the
// epilogue, and resets the counter. There is no spin-wait anywhere in this
// scheme.
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
  long long ld_out;
  float* slots;       // [2 * gridDim.x][NACC][128][MPAD] fp32 partial tiles
  int* counters;      // [row tiles] reduction blocks whose partials are in the slots; zero on entry and on exit
  int* done;          // [row tiles] contributors that have finished their share of the sum; zero likewise
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
// One CTA per SM. What the tails of these kernels cost (the time from a CTA's last MMA
// to its exit: publish partial tiles, wait for the other contributors, sum a share) was
// measured by removing all of it: 211 us at every M for K=8192, N=28672 against 222 us
// (M=8) and 245 us (M=64) with it. Tried against that gap and measured no better: two
// CTAs per SM with half the ring each (all CTAs reach their tails together, so there is
// no sibling stream to hide a tail behind); whole row tiles owned by CTAs with only the
// remainder split and summed early (15 us slower); the gate/up kernel prefetching the
// down projection's first weight boxes into L2 during its tail (no change).

// Weight sub-tiles (128 rows each) per work unit; they share the unit's activation
// tile. One is what ships. Two (gate/up) and four (down projection) sub-tiles at
// MPAD = 64 were measured on the K=8192, N=28672 problem: they cut the activation
// bytes an SM takes in per weight byte from 8/32 and 8/16 to 8/64, but at 72 KB a
// stage only three stages fit, every row tile then has two to nine contributors with
// four times the partial-tile volume, and the forward took 264 us against 247 us.
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_subtiles() {
  return 1;
}
template <int MPAD, bool DUAL>
__host__ __device__ constexpr int decode_stage_bytes() {
  return (DUAL ? 2 : 1) * decode_subtiles<MPAD, DUAL>() * 16384 + MPAD * 128;
}
// As many stages as fit in shared memory: bytes in flight per SM are what hides the
// DRAM latency (with 8 stages of 16 KB the down-projection kernel streamed at 5.6 TB/s
// where the gate/up kernel, with 160 KB in flight, reached 6.4 TB/s).
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

template <int MPAD, bool DUAL, typename T>
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
  constexpr uint32_t W_BYTES = 128 * 128;  // one [128 x 64] 16-bit weight sub-tile
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
      auto load_weights = [&](long long u, int st) {
        const int tile = static_cast<int>(u / args.kbt);
        const int kb = static_cast<int>(u - static_cast<long long>(tile) * args.kbt);
        const uint32_t sw = smem_base + st * STAGE_BYTES;
        const uint32_t fb = full_bar(st);
        mbar_expect_tx(fb, STAGE_BYTES);
        // Rows past the end of the matrix (a last tile that is not full) arrive as zeros.
#pragma unroll
        for (int b = 0; b < TILE_ROWS / BOX_ROWS; ++b) {
          tma_load_2d_hint(sw + b * BOX_ROWS * 128, &tmW0, fb, kb * BK, tile * TILE_ROWS + b * BOX_ROWS, pol_w);
          if (DUAL)
            tma_load_2d_hint(sw + SUB * W_BYTES + b * BOX_ROWS * 128, &tmW1, fb, kb * BK,
                             tile * TILE_ROWS + b * BOX_ROWS, pol_w);
        }
      };
      auto load_act = [&](long long u, int st) {
        const int kb = static_cast<int>(u % args.kbt);
        tma_load_2d_hint(smem_base + st * STAGE_BYTES + ACT_OFF, &tmAct, full_bar(st), kb * BK, 0, pol_a);
      };
      long long u = u_begin;
      if (args.dependent) {
        // The weights do not depend on the preceding kernel: fill the ring with them while
        // that kernel's last CTAs are still running, then wait for it and add the
        // activations of the same stages.
        const long long n0 = (u_end - u_begin) < STAGES ? (u_end - u_begin) : STAGES;
        for (long long i = 0; i < n0; ++i) load_weights(u_begin + i, static_cast<int>(i));
        pdl_wait();
        for (long long i = 0; i < n0; ++i) load_act(u_begin + i, static_cast<int>(i));
        u = u_begin + n0;
        stage = static_cast<int>(n0 % STAGES);
        phase = (n0 == STAGES) ? 1u : 0u;
      }
      for (; u < u_end; ++u) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        load_weights(u, stage);
        load_act(u, stage);
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
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint32_t accum = (first && k == 0) ? 0u : 1u;
              umma_f16(d_tmem + (t * NACC) * MPAD, w0desc + static_cast<uint64_t>(2 * k),
                       xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
              if (DUAL)
                umma_f16(d_tmem + (t * NACC + 1) * MPAD, w1desc + static_cast<uint64_t>(2 * k),
                         xdesc + static_cast<uint64_t>(2 * k), args.idesc, accum);
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
    long long pending[2];  // row tiles this CTA holds a partial of: at most its first and its last
    int npending = 0;
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
      // take the same way out, so they agree on the outcome of the wait first. Every
      // warp reaches this barrier because its wait above is bounded.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abortp != 0) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + lane_addr;

      // One output chunk: tokens [m0, m0 + count) of weight row `wrow`.
      auto emit = [&](long long wrow, float b0, float b1, int m0, const float* first, const float* second,
                      int count) {
        if (wrow >= args.rows) return;
#pragma unroll
        for (int i = 0; i < count; ++i) {
          const int m = m0 + i;
          if (m < args.M) {
            float o;
            if (DUAL) {
              o = act_value(args.act, first[i] + b0) * (second[i] + b1);
            } else {
              o = first[i] + b0;
            }
            const long long oi = static_cast<long long>(m) * args.ld_out + wrow;
            if (!DUAL && residual) o += static_cast<float>(residual[oi]);
            out[oi] = static_cast<T>(o);
          }
        }
      };
      auto row_bias = [&](const T* bias, long long wrow) {
        return (bias && wrow < args.rows) ? static_cast<float>(bias[wrow]) : 0.f;
      };
      // Slot layout: float4 (sub-tile t, accumulator a, i, row) at index
      // ((t * NACC + a) * MPAD/4 + i) * 128 + row, so that the 32 lanes of a warp (32
      // consecutive rows) touch 512 contiguous bytes per access.
      const int which = (u == u_begin) ? 0 : 1;
      float4* const slot4 = reinterpret_cast<float4*>(args.slots + (2LL * blockIdx.x + which) * SLOT_FLOATS);

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
        if (complete) {
          const long long wrow = tile * TILE_ROWS + t * 128 + r_in_tile;
          emit(wrow, row_bias(bias0, wrow), DUAL ? row_bias(bias1, wrow) : 0.f, 0, v[0], v[NACC - 1], MPAD);
        } else {
          // this CTA's partial sub-tile goes to its own slot
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

      if (!complete) {
        // Publish this CTA's share of the row tile and move on; the sum over the
        // contributors is taken up after the last segment (below).
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (ep_tid == 0) atomicAdd(args.counters + tile, static_cast<int>(seg_end - u));
        pending[npending++] = tile;
      }
      u = seg_end;
      ++seg;
    }

    // ---- split row tiles: every contributor sums an equal share of the tile ----
    // All of this CTA's partials are published by now, so nobody waits for a CTA
    // that is itself waiting. Contributor j of c (in CTA order) takes chunks
    // [j * P / c, (j + 1) * P / c) of the tile's P chunks (a chunk = 128 rows x 8 or
    // 16 tokens of one sub-tile), waits until every contributor's partial has been
    // counted (they all finish at about the same time: the unit ranges are equal),
    // adds the slots in CTA order, which makes the result independent of arrival
    // order, and applies the epilogue. The last contributor to finish clears the
    // tile's counters for the next call.
    constexpr int CHUNK4 = NACC == 2 ? 2 : 4;          // float4 columns per chunk and accumulator
    constexpr int CH_PER_SUB = MPAD / (4 * CHUNK4);
    constexpr int CHUNKS = SUB * CH_PER_SUB;
    constexpr int FIX_STAGE_CAP = 64;                  // 16-byte pieces a thread stages at a time (128 KB in all)
    for (int pi = 0; pi < npending && *abortp == 0; ++pi) {
      const long long tile = pending[pi];
      const long long tile_begin = tile * args.kbt;
      const long long tile_end = tile_begin + args.kbt;
      const long long c_first = ((tile_begin + 1) * gridDim.x - 1) / total;
      const long long c_last = (tile_end * gridDim.x - 1) / total;
      const int nc = static_cast<int>(c_last - c_first + 1);
      const int j = static_cast<int>(blockIdx.x - c_first);
      if (ep_tid == 0) {
        const volatile int* cnt = args.counters + tile;
        const long long t0 = clock64();
        while (*cnt != args.kbt) {
          if (*abortp != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES) {
            abort_flag = 1;
            atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
            break;
          }
          __nanosleep(64);
        }
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abortp != 0) break;
      auto row_bias = [&](const T* bias, long long wrow) {
        return (bias && wrow < args.rows) ? static_cast<float>(bias[wrow]) : 0.f;
      };
      const int p_begin = j * CHUNKS / nc, p_end = (j + 1) * CHUNKS / nc;
      // The loads of a share are independent, and their latency is the kernel's tail, so
      // they are issued all at once: cp.async copies them into the operand ring, which is
      // idle by now (every MMA of this CTA has completed), each thread into a column of
      // its own, and the sums are then taken from shared memory in CTA order.
      auto slot_of = [&](long long c) -> const float4* {
        const int w = unit_start(c, total, gridDim.x) >= tile_begin ? 0 : 1;
        return reinterpret_cast<const float4*>(args.slots + (2LL * c + w) * SLOT_FLOATS);
      };
      auto stage_addr = [&](int k) { return smem_base + static_cast<uint32_t>(k * 128 + ep_tid) * 16u; };
      auto issue_items = [&](int k, const float4* s4, int t, int ch) {  // ITEM4 copies for one (chunk, contributor)
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
          for (int i = 0; i < CHUNK4; ++i)
            cp_async_16(stage_addr(k + a * CHUNK4 + i),
                        s4 + ((t * NACC + a) * (MPAD / 4) + ch * CHUNK4 + i) * 128 + r_in_tile);
      };
      auto add_items = [&](int k, float (&sum)[NACC][4 * CHUNK4]) {
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
          for (int i = 0; i < CHUNK4; ++i) {
            const float4 q = ld_shared_f4(stage_addr(k + a * CHUNK4 + i));
            sum[a][4 * i] += q.x;
            sum[a][4 * i + 1] += q.y;
            sum[a][4 * i + 2] += q.z;
            sum[a][4 * i + 3] += q.w;
          }
      };
      auto emit_chunk = [&](int pch, const float (&sum)[NACC][4 * CHUNK4]) {
        const int t = pch / CH_PER_SUB, ch = pch - t * CH_PER_SUB;
        const long long wrow = tile * TILE_ROWS + t * 128 + r_in_tile;
        if (wrow >= args.rows) return;
        const float b0 = row_bias(bias0, wrow);
        const float b1 = DUAL ? row_bias(bias1, wrow) : 0.f;
#pragma unroll
        for (int i = 0; i < 4 * CHUNK4; ++i) {
          const int m = ch * 4 * CHUNK4 + i;
          if (m < args.M) {
            float o;
            if (DUAL) {
              o = act_value(args.act, sum[0][i] + b0) * (sum[NACC - 1][i] + b1);
            } else {
              o = sum[0][i] + b0;
            }
            const long long oi = static_cast<long long>(m) * args.ld_out + wrow;
            if (!DUAL && residual) o += static_cast<float>(residual[oi]);
            out[oi] = static_cast<T>(o);
          }
        }
      };
      constexpr int ITEM4 = NACC * CHUNK4;  // 16-byte pieces per (chunk, contributor) and thread
      int pch = p_begin;
      while (pch < p_end) {
        if (nc * ITEM4 <= FIX_STAGE_CAP) {
          // several chunks, all their contributors, in one round trip
          int nch = FIX_STAGE_CAP / (nc * ITEM4);
          if (nch > p_end - pch) nch = p_end - pch;
          int k = 0;
          for (int q = 0; q < nch; ++q) {
            const int t = (pch + q) / CH_PER_SUB, ch = (pch + q) - t * CH_PER_SUB;
            for (long long c = c_first; c <= c_last; ++c, k += ITEM4) issue_items(k, slot_of(c), t, ch);
          }
          cp_async_wait_all();
          k = 0;
          for (int q = 0; q < nch; ++q) {
            float sum[NACC][4 * CHUNK4];
#pragma unroll
            for (int a = 0; a < NACC; ++a)
#pragma unroll
              for (int i = 0; i < 4 * CHUNK4; ++i) sum[a][i] = 0.f;
            for (int ci = 0; ci < nc; ++ci, k += ITEM4) add_items(k, sum);
            emit_chunk(pch + q, sum);
          }
          pch += nch;
        } else {
          // one chunk, its many contributors in batches
          const int t = pch / CH_PER_SUB, ch = pch - t * CH_PER_SUB;
          float sum[NACC][4 * CHUNK4];
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int i = 0; i < 4 * CHUNK4; ++i) sum[a][i] = 0.f;
          constexpr int CB = FIX_STAGE_CAP / ITEM4;
          for (long long cb = c_first; cb <= c_last; cb += CB) {
            const long long ce = cb + CB - 1 < c_last ? cb + CB - 1 : c_last;
            int k = 0;
            for (long long c = cb; c <= ce; ++c, k += ITEM4) issue_items(k, slot_of(c), t, ch);
            cp_async_wait_all();
            k = 0;
            for (long long c = cb; c <= ce; ++c, k += ITEM4) add_items(k, sum);
          }
          emit_chunk(pch, sum);
          pch += 1;
        }
      }
      // Everybody has read what it needs of this tile's slots: count this CTA as done.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ep_tid == 0) {
        __threadfence();
        if (atomicAdd(args.done + tile, 1) == nc - 1) {
          args.counters[tile] = 0;  // leave the scratch ready for the next call
          args.done[tile] = 0;
        }
      }
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
