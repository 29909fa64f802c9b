// One-launch decode forward: y = (act(x Wg^T + bg) * (x Wu^T + bu)) Wd^T + bd (+ residual) for
// M <= 64 tokens, with BOTH weight streams in one persistent kernel (16-bit weights).
//
// The work is that of the two kernels of decode_stream.cuh, with the same swap-AB tiles and
// the same stream-K split of each matrix over the CTAs; what differs is how the second stream
// follows the first. Every CTA walks ONE operand ring through both phases:
//
//   phase 1  unit = (128 rows of W_gate and W_up, 64 reduction columns); two ring slots, the
//            first with the W_gate tile and the activation block of x, the second with the
//            W_up tile; two accumulators; the epilogue writes H.
//   phase 2  unit = (128 rows of W_down, 64 reduction columns); one slot with the weight tile
//            and the activation block of H; one accumulator; the epilogue writes y.
//
// A slot is [16 KB of weights][MPAD x 128 B of activations] in both phases, so the producer
// runs on from the last tile of W_gate / W_up into W_down without draining the ring: the
// weight stream never stops between the projections, and there is no second launch, no second
// barrier / TMEM set-up and no drain of the grid in between. Phase 2 reads H, which every CTA
// of the grid has a share in: the CTA that completes a row tile of phase 1 (= 128 columns of
// H) adds one to a device-wide count with release semantics, and a producer issues the H
// blocks of its phase-2 slots only once that count has reached the number of row tiles
// (acquire + proxy fence, since the blocks are then read by TMA). Until then it keeps
// streaming W_down tiles into free slots and remembers which slots still lack their
// activations; if the whole ring is in that state it waits (bounded) for the count.
//
// Who waits for whom: owners of split row tiles wait for the other contributors' partials, as
// in decode_stream.cuh (contributors never wait before they publish); phase 2 of any CTA waits
// for phase 1 of all CTAs, and phase 1 waits for nothing in phase 2. The grid is at most one
// CTA per SM, so all CTAs are resident unless another kernel holds SMs; in that case the waits
// run out after WAIT_LIMIT_CYCLES, the status word is set and the output is incomplete.
// The last CTA to finish clears the two device-wide counts for the next call.
#pragma once
#include "decode_stream.cuh"

namespace gmlp {

struct DecodeFusedArgs {
  int M;  // tokens (<= MPAD)
  int N;  // intermediate size: weight rows of phase 1, reduction length of phase 2
  int K;  // hidden size: reduction length of phase 1, weight rows of phase 2
  uint32_t idesc;
  int* status;
  const void* b_gate;
  const void* b_up;
  const void* b_down;
  void* h;                 // [M, N]
  void* y;                 // [M, K]
  const void* residual;    // optional [M, K]
  const float* row_scale;  // optional [M] per-token factors on the phase-1 accumulators
  float* slots;            // [2 * gridDim.x][2][128][MPAD] fp32: CTA c uses slot 2c in phase 1, 2c+1 in phase 2
  int* counters1;          // [row tiles of phase 1]; zero on entry and on exit (unless a wait was given up)
  int* counters2;          // [row tiles of phase 2]; the same
  int* sync;               // [0] row tiles of phase 1 whose columns of H are complete, [1] CTAs that are done
  int act;
  int dependent;           // launched with programmatic stream serialization
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int MPAD>
__host__ __device__ constexpr int fused_slot_bytes() { return 16384 + MPAD * 128; }
template <int MPAD>
__host__ __device__ constexpr int fused_stages() {
  constexpr int fit = (232448 - 1024 - 512) / fused_slot_bytes<MPAD>();
  return fit > 12 ? 12 : fit;
}
template <int MPAD>
constexpr size_t fused_smem_bytes() {
  return static_cast<size_t>(fused_stages<MPAD>()) * fused_slot_bytes<MPAD>() + 1024;
}

// What the epilogue warps need to know about one phase.
struct FusedPhase {
  int rows;             // weight rows
  int kbt;              // reduction blocks per row tile
  long long u_begin, u_end, total;
  void* out;            // [M, rows]
  const void* bias0;
  const void* bias1;
  const void* residual;
  const float* row_scale;
  int* counters;
  float* slot;          // this CTA's partial-tile slot for the phase
};

// The epilogue warps' walk over one phase's segments. Returns false when a wait was given up
// (all four warps return the same answer). `seg` runs on across the phases.
template <int MPAD, bool DUAL, typename T, int STAGES>
__device__ __forceinline__ bool fused_epilogue_phase(const DecodeFusedArgs& args, const FusedPhase& ph, int& seg,
                                                     uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
                                                     uint32_t smem_base, volatile int* abortp, int* abort_flag) {
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr uint32_t ACC_COLS = 2 * MPAD;  // columns per accumulator buffer, both phases
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int quarter = warp & 3;
  const int r_in_tile = quarter * 32 + lane;
  const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
  const int ep_tid = threadIdx.x - 64;
  T* const out = static_cast<T*>(ph.out);
  const T* const residual = static_cast<const T*>(ph.residual);
  const T* const bias0 = static_cast<const T*>(ph.bias0);
  const T* const bias1 = static_cast<const T*>(ph.bias1);
  const long long ld_out = ph.rows;

  long long u = ph.u_begin;
  while (u < ph.u_end) {
    const long long tile = u / ph.kbt;
    const long long tile_begin = tile * ph.kbt;
    const long long tile_end = tile_begin + ph.kbt;
    const long long seg_end = tile_end < ph.u_end ? tile_end : ph.u_end;
    const bool complete = (u == tile_begin) && (seg_end == tile_end);
    const int acc = seg & 1;
    const uint32_t acc_phase = (seg >> 1) & 1;
    const bool got = mbar_wait_warp(tfull0 + 8u * acc, acc_phase, abortp, lane);
    if (!got && lane == 0) {
      *abort_flag = 1;
      atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
    }
    // one answer for all four warps, whenever the abort flag flips
    if (named_bar_or(1, 128, *abortp != 0)) return false;
    tc_fence_after_sync();
    const uint32_t taddr = tmem_base + acc * ACC_COLS + lane_addr;

    const bool owner = !complete && (u == tile_begin);
    const long long c_first = ((tile_begin + 1) * gridDim.x - 1) / ph.total;
    const long long c_last = (tile_end * gridDim.x - 1) / ph.total;
    if (owner) {
      if (ep_tid == 0) {
        const int need = ph.kbt - static_cast<int>(seg_end - u);
        const volatile int* cnt = ph.counters + tile;
        const long long t0 = clock64();
        while (*cnt != need) {
          if (*abortp != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_EPILOGUE);
            break;
          }
          __nanosleep(64);
        }
        __threadfence();
      }
      if (named_bar_or(1, 128, *abortp != 0)) return false;
    }

    float v[NACC][MPAD];
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
#pragma unroll
      for (int c = 0; c < MPAD / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x16(taddr + a * MPAD + c * 16, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) v[a][c * 16 + i] = __uint_as_float(r[i]);
      }
    }
    // TMEM has been read into registers: the MMA issuer may reuse the buffer.
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(tempty0 + 8u * acc);

    if (owner) {
      // The other contributors' parts, added in CTA order. In phase 2 this is the CTA's last
      // segment and the ring is idle, so the parts come in through it with asynchronous copies,
      // as many contributors per round trip as it holds; in phase 1 the ring already carries
      // W_down tiles, and the parts are read straight from L2.
      constexpr int ITEM4 = NACC * (MPAD / 4);
      if (DUAL) {
        for (long long c = c_first + 1; c <= c_last; ++c) {
          const float4* s4 = reinterpret_cast<const float4*>(args.slots + (2LL * c) * (2LL * 128 * MPAD));
          // eight 16-byte loads in flight per thread at a time (more would not fit the registers)
          constexpr int CH = (MPAD / 4) < 8 ? (MPAD / 4) : 8;
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int i0 = 0; i0 < MPAD / 4; i0 += CH) {
              float4 q[CH];
#pragma unroll
              for (int j = 0; j < CH; ++j) q[j] = __ldcg(s4 + (a * (MPAD / 4) + i0 + j) * 128 + r_in_tile);
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                v[a][4 * (i0 + j)] += q[j].x;
                v[a][4 * (i0 + j) + 1] += q[j].y;
                v[a][4 * (i0 + j) + 2] += q[j].z;
                v[a][4 * (i0 + j) + 3] += q[j].w;
              }
            }
        }
      } else {
        constexpr int RING_CAP = STAGES * fused_slot_bytes<MPAD>() / (128 * 16);
        constexpr int FIX_CONTRIB = RING_CAP / ITEM4;
        static_assert(ITEM4 <= RING_CAP, "the ring must hold one contributor's part");
        auto stage_addr = [&](int k) { return smem_base + static_cast<uint32_t>(k * 128 + ep_tid) * 16u; };
        for (long long cb = c_first + 1; cb <= c_last; cb += FIX_CONTRIB) {
          const long long ce = cb + FIX_CONTRIB - 1 < c_last ? cb + FIX_CONTRIB - 1 : c_last;
          int k = 0;
          for (long long c = cb; c <= ce; ++c) {
            const float4* s4 = reinterpret_cast<const float4*>(args.slots + (2LL * c + 1) * (2LL * 128 * MPAD));
#pragma unroll
            for (int i = 0; i < ITEM4; ++i, ++k) cp_async_16(stage_addr(k), s4 + i * 128 + r_in_tile);
          }
          cp_async_wait_all();
          k = 0;
          for (long long c = cb; c <= ce; ++c) {
#pragma unroll
            for (int i = 0; i < MPAD / 4; ++i, ++k) {
              const float4 q = ld_shared_f4(stage_addr(k));
              v[0][4 * i] += q.x;
              v[0][4 * i + 1] += q.y;
              v[0][4 * i + 2] += q.z;
              v[0][4 * i + 3] += q.w;
            }
          }
        }
      }
    }

    if (complete || owner) {
      const long long wrow = tile * 128 + r_in_tile;
      if (wrow < ph.rows) {
        const float b0 = bias0 ? static_cast<float>(bias0[wrow]) : 0.f;
        T* const po = out + wrow;
        if (DUAL) {
          const float b1 = bias1 ? static_cast<float>(bias1[wrow]) : 0.f;
          const bool scaled = ph.row_scale != nullptr;
          const float* g = v[0];
          const float* up = v[NACC - 1];
          switch (args.act) {  // chosen outside the unrolled token loop
            case ACT_SILU: store_gated<ACT_SILU, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            case ACT_NONE: store_gated<ACT_NONE, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            case ACT_RELU: store_gated<ACT_RELU, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            case ACT_GELU: store_gated<ACT_GELU, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            case ACT_SIGMOID: store_gated<ACT_SIGMOID, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            case ACT_TANH: store_gated<ACT_TANH, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
            default: store_gated<ACT_LEAKY_RELU, MPAD>(po, ld_out, args.M, g, up, b0, b1, ph.row_scale, scaled, 1.f, 1.f); break;
          }
        } else {
          const T* const pr = residual ? residual + wrow : nullptr;
#pragma unroll
          for (int m = 0; m < MPAD; ++m) {
            if (m < args.M) {
              float o = v[0][m] + b0;
              if (pr) o += static_cast<float>(pr[static_cast<long long>(m) * ld_out]);
              po[static_cast<long long>(m) * ld_out] = static_cast<T>(o);
            }
          }
        }
      }
      if (owner && ep_tid == 0) ph.counters[tile] = 0;  // leave the scratch ready for the next call
      if (DUAL) {
        // 128 more columns of H are complete: make them visible to the TMA reads of every CTA's
        // phase 2, then count the tile.
        fence_proxy_async_all();
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) red_release_gpu_add(args.sync, 1);
      }
    } else {
      // this CTA's part of the tile goes to its slot: float4 (accumulator a, i, row) at index
      // (a * MPAD/4 + i) * 128 + row, 512 contiguous bytes per warp and access
      float4* const slot4 = reinterpret_cast<float4*>(ph.slot);
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int i = 0; i < MPAD / 4; ++i)
          slot4[(a * (MPAD / 4) + i) * 128 + r_in_tile] =
              make_float4(v[a][4 * i], v[a][4 * i + 1], v[a][4 * i + 2], v[a][4 * i + 3]);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ep_tid == 0) atomicAdd(ph.counters + tile, static_cast<int>(seg_end - u));
    }
    u = seg_end;
    ++seg;
  }
  return true;
}

template <int MPAD, typename T>
__global__ void __launch_bounds__(DECODE_THREADS, 1)
decode_fused_kernel(const __grid_constant__ CUtensorMap tmWg, const __grid_constant__ CUtensorMap tmWu,
                    const __grid_constant__ CUtensorMap tmWd, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmH, const DecodeFusedArgs args) {
  static_assert(MPAD == 16 || MPAD == 32 || MPAD == 64, "token padding");
  constexpr int STAGES = fused_stages<MPAD>();
  static_assert(STAGES >= 4, "phase 1 takes two slots per unit");
  constexpr uint32_t W_BYTES = 128 * 128;
  constexpr uint32_t ACT_BYTES = MPAD * 128;
  constexpr uint32_t SLOT_BYTES = W_BYTES + ACT_BYTES;
  static_assert(SLOT_BYTES == fused_slot_bytes<MPAD>(), "slot layout");
  constexpr uint32_t ACC_COLS = 2 * MPAD;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;  // 64, 128 or 256

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t tfull0 = bar_base + 8u * (2 * STAGES);
  const uint32_t tempty0 = bar_base + 8u * (2 * STAGES + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kbt1 = args.K / BK, kbt2 = args.N / BK;
  const long long tiles1 = (args.N + 127) / 128, tiles2 = (args.K + 127) / 128;
  const long long total1 = tiles1 * kbt1, total2 = tiles2 * kbt2;
  const long long u1_begin = unit_start(blockIdx.x, total1, gridDim.x);
  const long long u1_end = unit_start(blockIdx.x + 1, total1, gridDim.x);
  const long long u2_begin = unit_start(blockIdx.x, total2, gridDim.x);
  const long long u2_end = unit_start(blockIdx.x + 1, total2, gridDim.x);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8u * a, 1);
      mbar_init(tempty0 + 8u * a, 4);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmWg);
    tma_prefetch_desc(&tmWu);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmWd);
    tma_prefetch_desc(&tmH);
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
      const uint64_t pol_w = l2_policy_evict_first();  // weights are read once
      const uint64_t pol_a = l2_policy_evict_last();   // activations by every CTA
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto next = [&]() {
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      };
      auto slot_addr = [&](int s) { return smem_base + static_cast<uint32_t>(s) * SLOT_BYTES; };
      // phase 1, unit u in slots s0 (W_gate + x) and s1 (W_up)
      // (row tile, reduction block) of the next unit to issue, per stream, kept incrementally: a 64-bit
      // division per unit would cost the issuing thread a good part of the time a 16 KB unit takes to stream
      int w_tile = static_cast<int>(u1_begin / kbt1);
      int w_kb = static_cast<int>(u1_begin - static_cast<long long>(w_tile) * kbt1);
      int a_kb = w_kb;
      auto load_w1 = [&](int s0, int s1) {
        const int tile = w_tile, kb = w_kb;
        if (++w_kb == kbt1) {
          w_kb = 0;
          ++w_tile;
        }
        mbar_expect_tx(full_bar(s0), SLOT_BYTES);
        tma_load_2d_hint(slot_addr(s0), &tmWg, full_bar(s0), kb * BK, tile * 128, pol_w);
        mbar_expect_tx(full_bar(s1), W_BYTES);
        tma_load_2d_hint(slot_addr(s1), &tmWu, full_bar(s1), kb * BK, tile * 128, pol_w);
      };
      auto load_x = [&](int s0) {
        const int kb = a_kb;
        if (++a_kb == kbt1) a_kb = 0;
        tma_load_2d_hint(slot_addr(s0) + W_BYTES, &tmX, full_bar(s0), kb * BK, 0, pol_a);
      };
      auto load_w2 = [&](int s) {
        const int tile = w_tile, kb = w_kb;
        if (++w_kb == kbt2) {
          w_kb = 0;
          ++w_tile;
        }
        mbar_expect_tx(full_bar(s), SLOT_BYTES);
        tma_load_2d_hint(slot_addr(s), &tmWd, full_bar(s), kb * BK, tile * 128, pol_w);
      };
      auto load_h = [&](int s) {  // blocks of H go out in unit order, so the count runs on
        const int kb = a_kb;
        if (++a_kb == kbt2) a_kb = 0;
        tma_load_2d_hint(slot_addr(s) + W_BYTES, &tmH, full_bar(s), kb * BK, 0, pol_a);
      };

      // ---- phase 1
      long long u = u1_begin;
      if (args.dependent) {
        // The weights do not depend on the preceding kernel: fill the ring with them while that
        // kernel's last CTAs are still running, then wait for it and add the activations.
        const long long left = u1_end - u1_begin;
        const long long n0 = left < STAGES / 2 ? left : STAGES / 2;
        for (long long i = 0; i < n0; ++i) load_w1(static_cast<int>(2 * i), static_cast<int>(2 * i + 1));
        pdl_wait();
        for (long long i = 0; i < n0; ++i) load_x(static_cast<int>(2 * i));
        u = u1_begin + n0;
        for (long long i = 0; i < 2 * n0; ++i) next();
      }
      for (; u < u1_end; ++u) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        const int s0 = stage;
        next();
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
          ok = false;
          break;
        }
        const int s1 = stage;
        next();
        load_w1(s0, s1);
        load_x(s0);
      }

      // ---- phase 2: W_down tiles at once, their blocks of H when all of H is there
      int pending = 0;  // the last `pending` units' slots hold weights but lack activations
      bool h_ready = false;
      auto h_poll = [&]() {
        if (ld_acquire_gpu(args.sync) < static_cast<int>(tiles1)) return false;
        fence_proxy_async_all();
        return true;
      };
      auto h_wait = [&]() {
        const long long t0 = clock64();
        while (!h_poll()) {
          if (*abortp != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
          __nanosleep(200);
        }
        return true;
      };
      auto flush = [&]() {  // the last `pending` units sit in the slots before `stage`, oldest first
        for (int i = pending; i >= 1; --i) load_h((stage - i + 2 * STAGES) % STAGES);
        pending = 0;
      };
      w_tile = static_cast<int>(u2_begin / kbt2);
      w_kb = static_cast<int>(u2_begin - static_cast<long long>(w_tile) * kbt2);
      a_kb = w_kb;
      if (ok) {
        for (u = u2_begin; u < u2_end; ++u) {
          if (!h_ready && pending == STAGES) {  // the slot to reuse is itself waiting for H
            if (!h_wait()) {
              ok = false;
              break;
            }
            h_ready = true;
            flush();
          }
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abortp)) {
            ok = false;
            break;
          }
          load_w2(stage);
          if (!h_ready) h_ready = h_poll();
          if (h_ready) {
            flush();
            load_h(stage);
          } else {
            ++pending;
          }
          next();
        }
        if (ok && pending > 0) {
          if (h_wait()) {
            flush();
          } else {
            ok = false;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_PRODUCER);
        // Copies issued a moment ago may still be on their way into the ring: give them time
        // to land before the CTA (and its shared memory) goes away.
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int seg = 0;
      bool ok = true;
      auto next = [&]() {
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      };
      auto slot_addr = [&](int s) { return smem_base + static_cast<uint32_t>(s) * SLOT_BYTES; };
      auto mma4 = [&](uint32_t d, uint32_t w_addr, uint32_t x_addr, bool first) {
        const uint64_t wdesc = make_smem_desc(w_addr, 16, 1024);
        const uint64_t xdesc = make_smem_desc(x_addr, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(d, wdesc + static_cast<uint64_t>(2 * k), xdesc + static_cast<uint64_t>(2 * k), args.idesc,
                   (first && k == 0) ? 0u : 1u);
      };
      for (int p = 0; p < 2 && ok; ++p) {
        const int kbt = p == 0 ? kbt1 : kbt2;
        long long u = p == 0 ? u1_begin : u2_begin;
        const long long u_end = p == 0 ? u1_end : u2_end;
        while (u < u_end && ok) {
          const long long tile = u / kbt;
          const long long tile_end = (tile + 1) * kbt;
          const long long seg_end = tile_end < u_end ? tile_end : u_end;
          const int acc = seg & 1;
          const uint32_t acc_phase = (seg >> 1) & 1;
          if (!mbar_wait(tempty0 + 8u * acc, acc_phase ^ 1u, abortp)) {
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
            const int s0 = stage;
            next();
            mma4(d_tmem, slot_addr(s0), slot_addr(s0) + W_BYTES, first);
            if (p == 0) {
              if (!mbar_wait(full_bar(stage), phase, abortp)) {
                ok = false;
                break;
              }
              tc_fence_after_sync();
              const int s1 = stage;
              next();
              mma4(d_tmem + MPAD, slot_addr(s1), slot_addr(s0) + W_BYTES, first);
              umma_commit(empty_bar(s0));
              umma_commit(empty_bar(s1));
            } else {
              umma_commit(empty_bar(s0));
            }
            first = false;
          }
          if (ok) umma_commit(tfull0 + 8u * acc);
          ++seg;
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(args.status, 0, GMLP_DEV_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    if (args.dependent) pdl_wait();  // slots, counters and outputs may still be in use by the preceding grid
    int seg = 0;
    FusedPhase p1;
    p1.rows = args.N;
    p1.kbt = kbt1;
    p1.u_begin = u1_begin;
    p1.u_end = u1_end;
    p1.total = total1;
    p1.out = args.h;
    p1.bias0 = args.b_gate;
    p1.bias1 = args.b_up;
    p1.residual = nullptr;
    p1.row_scale = args.row_scale;
    p1.counters = args.counters1;
    p1.slot = args.slots + (2LL * blockIdx.x) * (2LL * 128 * MPAD);
    if (fused_epilogue_phase<MPAD, true, T, STAGES>(args, p1, seg, tmem_base, tfull0, tempty0, smem_base, abortp,
                                                    &abort_flag)) {
      FusedPhase p2;
      p2.rows = args.K;
      p2.kbt = kbt2;
      p2.u_begin = u2_begin;
      p2.u_end = u2_end;
      p2.total = total2;
      p2.out = args.y;
      p2.bias0 = args.b_down;
      p2.bias1 = nullptr;
      p2.residual = args.residual;
      p2.row_scale = nullptr;
      p2.counters = args.counters2;
      p2.slot = args.slots + (2LL * blockIdx.x + 1) * (2LL * 128 * MPAD);
      fused_epilogue_phase<MPAD, false, T, STAGES>(args, p2, seg, tmem_base, tfull0, tempty0, smem_base, abortp,
                                                   &abort_flag);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) {
    // The CTA that finds all the others done has nobody left to disturb: it clears the
    // device-wide counts for the next call. (This thread is the producer: it has passed its wait
    // for the preceding grid, so these are this call's counts.)
    __threadfence();
    const int done = atomicAdd(args.sync + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      args.sync[0] = 0;
      args.sync[1] = 0;
    }
  }
}

}  // namespace gmlp
