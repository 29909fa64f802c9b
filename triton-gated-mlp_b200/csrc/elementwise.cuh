// HBM-bound helper kernels around the GEMMs: the SiLU/multiply derivative for a
// caller-supplied dH, column sums for the bias gradients, and the dropout-mask
// dump used by the bit-exact mask check.
#pragma once
#include <cuda_fp8.h>

#include "gemm_tcgen05.cuh"

namespace gmlp {

// d_gate = dH' * u * act'(g), d_up = dH' * act(g), dH' = dH * keep / (1-p).
// One thread per 8 consecutive columns; grid-stride over the [M, N] matrix.
template <typename T>
__global__ void __launch_bounds__(256)
dact_kernel(const T* __restrict__ dh, const T* __restrict__ g, const T* __restrict__ u,
            T* __restrict__ d_gate, T* __restrict__ d_up, long long M, long long N,
            DropoutParams drop, int act) {
  const long long groups_per_row = N / 8;
  const long long total = M * groups_per_row;
  const bool drop_on = drop.thresh != 0u;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / groups_per_row;
    const long long col = (i - row * groups_per_row) * 8;
    const long long o = row * N + col;
    float a[8], gv[8], uv[8], dg[8], du[8];
    load8(dh + o, a);
    load8(g + o, gv);
    load8(u + o, uv);
    if (drop_on) {
      float f[8];
      dropout_factors8(drop, drop.row0_global + row, drop.col0_global + col, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] *= f[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float f, df;
      act_value_grad(act, gv[k], f, df);
      du[k] = a[k] * f;
      dg[k] = a[k] * uv[k] * df;
    }
    store8(d_gate + o, dg);
    store8(d_up + o, du);
  }
}

// keep-mask dump: one thread per 8 consecutive columns.
__global__ void __launch_bounds__(256)
dropout_mask_kernel(uint8_t* __restrict__ mask, long long M, long long N, DropoutParams drop) {
  const long long groups_per_row = N / 8;
  const long long total = M * groups_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / groups_per_row;
    const long long col = (i - row * groups_per_row) * 8;
    float f[8];
    dropout_factors8(drop, drop.row0_global + row, drop.col0_global + col, f);
    uint2 m;
    m.x = (f[0] != 0.f) | ((f[1] != 0.f) << 8) | ((f[2] != 0.f) << 16) | ((f[3] != 0.f) << 24);
    m.y = (f[4] != 0.f) | ((f[5] != 0.f) << 8) | ((f[6] != 0.f) << 16) | ((f[7] != 0.f) << 24);
    *reinterpret_cast<uint2*>(mask + row * N + col) = m;
  }
}

// RMSNorm ahead of the MLP (the step before it in a Llama block). One warp per token row.
//   rs[m] = 1 / sqrt(mean_k x[m,k]^2 + eps)          (fp32)
//   xn[m,k] = x[m,k] * rs[m]                         (optional, in x's type)
// The forward pass needs only rs: the gate/up kernel multiplies its accumulators by rs[row]
// (the norm's weight is folded into W_gate / W_up), so the normalised activations are never
// written. Training keeps xn for the backward pass below.
template <typename T>
__global__ void __launch_bounds__(256)
rms_rowscale_kernel(const T* __restrict__ x, long long M, long long K, long long ld, float eps,
                    float* __restrict__ rs, T* __restrict__ xn) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= M) return;
  const T* xr = x + row * ld;
  float ss = 0.f;
  for (long long k = lane * 8LL; k < K; k += 256) {
    float v[8];
    load8(xr + k, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss / static_cast<float>(K) + eps);
  if (lane == 0) rs[row] = r;
  if (xn != nullptr) {
    T* out = xn + row * K;
    for (long long k = lane * 8LL; k < K; k += 256) {
      float v[8];
      load8(xr + k, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= r;
      store8(out + k, v);
    }
  }
}

// Backward of xn = x * rs: dx[m,:] = rs[m] * (dxn[m,:] - xn[m,:] * mean_k(dxn[m,k] * xn[m,k])).
template <typename T>
__global__ void __launch_bounds__(256)
rms_bwd_kernel(const T* __restrict__ dxn, const T* __restrict__ xn, const float* __restrict__ rs,
               long long M, long long K, T* __restrict__ dx) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= M) return;
  const T* a = dxn + row * K;
  const T* b = xn + row * K;
  float dot = 0.f;
  for (long long k = lane * 8LL; k < K; k += 256) {
    float u[8], v[8];
    load8(a + k, u);
    load8(b + k, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) dot = fmaf(u[i], v[i], dot);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  const float c = dot / static_cast<float>(K), r = rs[row];
  T* out = dx + row * K;
  for (long long k = lane * 8LL; k < K; k += 256) {
    float u[8], v[8];
    load8(a + k, u);
    load8(b + k, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) u[i] = r * (u[i] - v[i] * c);
    store8(out + k, u);
  }
}

// Per-row dynamic quantisation to e4m3 for the 8-bit decode path. One 256-thread block per row
// (the decode path has at most 64 rows, each up to tens of thousands of elements long):
//   scale[m] = max(amax_k |x[m,k]|, tiny) / 448       (448 = largest e4m3 value)
//   q[m,k]   = e4m3(x[m,k] / scale[m]), round to nearest even, saturating
// so that x ~= q * scale. The CPU restatement is oracle/fp8.py.
// `dependent`: launched as a programmatic dependent of the kernel that writes x. The grid lets
// ITS dependent (a weight-streaming kernel) start at once and waits for x's producer itself.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_e4m3_kernel(const T* __restrict__ x, long long M, long long K, long long ld,
                          uint8_t* __restrict__ q, float* __restrict__ scale, int dependent) {
  __shared__ float warp_max[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (dependent) asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31;
  const T* xr = x + row * ld;
  float amax = 0.f;
  for (long long k = tid * 8LL; k < K; k += 2048) {
    float v[8];
    load8(xr + k, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) warp_max[tid >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, warp_max[w]);
  const float sc = fmaxf(amax, 1e-30f) / 448.0f;
  if (tid == 0) scale[row] = sc;
  uint8_t* out = q + row * K;
  for (long long k = tid * 8LL; k < K; k += 2048) {
    float v[8];
    load8(xr + k, v);
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // true division, so that the CPU restatement (which divides) agrees bit for bit
      const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h] / sc, v[4 * h + 1] / sc),
                                                               __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * h + 2] / sc, v[4 * h + 3] / sc),
                                                               __NV_SATFINITE, __NV_E4M3);
      w[h] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    *reinterpret_cast<uint2*>(out + k) = make_uint2(w[0], w[1]);
  }
}

// Column sums, pass 1: block (cb, rb) sums rows [rb*rows_per_block, ...) of the
// 128 columns starting at cb*128 and writes them to partial[rb, :].
constexpr int COLSUM_COLS = 128;
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ src, long long rows, long long cols, long long ld,
                      long long rows_per_block, float* __restrict__ partial) {
  __shared__ float red[16][COLSUM_COLS + 4];
  const int tx = threadIdx.x & 15;  // 8-column group inside the 128-column slab
  const int ty = threadIdx.x >> 4;  // row lane
  const long long col = static_cast<long long>(blockIdx.x) * COLSUM_COLS + tx * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
    for (long long r = r0 + ty; r < r1; r += 16) {
      float v[8];
      load8(src + r * ld + col, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[ty][tx * 8 + k] = acc[k];
  __syncthreads();
  if (threadIdx.x < COLSUM_COLS) {
    const long long c = static_cast<long long>(blockIdx.x) * COLSUM_COLS + threadIdx.x;
    if (c < cols) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) s += red[j][threadIdx.x];
      partial[static_cast<long long>(blockIdx.y) * cols + c] = s;
    }
  }
}

// Column sums, pass 2: dst[c] = sum_rb partial[rb, c], rounded to T.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, long long cols, int row_blocks,
                    T* __restrict__ dst) {
  const long long c = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int rb = 0; rb < row_blocks; ++rb) s += partial[static_cast<long long>(rb) * cols + c];
  dst[c] = static_cast<T>(s);
}

}  // namespace gmlp
