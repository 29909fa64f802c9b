// C ABI of libgmlp.so (declared in include/gmlp.h): argument checks, TMA tensor
// map encoding and kernel launches. No torch types, no allocation, no CPU path.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/gmlp.h"
#include "decode_stream.cuh"
#include "decode_fused.cuh"
#include "elementwise.cuh"
#include "gemm_tcgen05.cuh"
#include "peer_reduce.cuh"

namespace gmlp {

// ------------------------------------------------------------------ errors --
static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// Per-device status word written by kernels that give up a bounded wait.
__device__ int g_dev_status;

struct DeviceInfo {
  std::atomic<bool> ready{false};
  int sm_count = 0;
  int cc_major = 0;
  int* status_ptr = nullptr;
};
static DeviceInfo g_dev[64];
static std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int device_info(const DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(GMLP_ERR_ARG, "device index %d out of range", dev);
  // Binds the device's primary context to the calling thread. Threads that never
  // made a runtime call that needs a context (autograd's backward threads) have the
  // right device selected but no driver context, which tensor-map encoding needs.
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaSetDevice: %s", cudaGetErrorString(e));
  DeviceInfo& d = g_dev[dev];
  if (d.ready.load(std::memory_order_acquire)) {
    *out = &d;
    return GMLP_OK;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!d.ready.load(std::memory_order_relaxed)) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess)
      return fail(GMLP_ERR_LAUNCH, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    d.sm_count = prop.multiProcessorCount;
    d.cc_major = prop.major;
    if (d.cc_major != 10)
      return fail(GMLP_ERR_ARCH, "libgmlp needs an sm_100a device, found compute capability %d.%d",
                  prop.major, prop.minor);
    void* sp = nullptr;
    e = cudaGetSymbolAddress(&sp, g_dev_status);
    if (e != cudaSuccess)
      return fail(GMLP_ERR_LAUNCH, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    d.status_ptr = static_cast<int*>(sp);
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess)
        return fail(GMLP_ERR_LAUNCH, "cuTensorMapEncodeTiled entry point not available");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    d.ready.store(true, std::memory_order_release);
  }
  *out = &d;
  return GMLP_OK;
}

// ------------------------------------------------------------- tensor maps --
// Encoded maps are kept in a small per-thread cache keyed by everything that goes
// into the encoding: a training loop presents the same (pointer, shape) pairs step
// after step (weights always, activations whenever the allocator hands the same
// blocks back), and cuTensorMapEncodeTiled is a driver call of about a microsecond.
// A map holds no reference to the memory it describes, so a stale entry whose key
// matches again is exactly the map a fresh encoding would give. Per thread: no lock,
// and calls from different host threads never share an entry.
struct MapKey {
  const void* base;
  int64_t inner, outer, pitch;
  uint32_t box_inner, box_outer;
  int32_t dtype, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && pitch == o.pitch &&
           box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype &&
           swizzle == o.swizzle;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int MAP_CACHE_SLOTS = 256;
static thread_local MapSlot g_map_cache[MAP_CACHE_SLOTS];

static uint32_t map_hash(const MapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.inner) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.outer) * 0x165667B19E3779F9ull;
  h ^= (static_cast<uint64_t>(k.box_inner) << 40) ^ (static_cast<uint64_t>(k.box_outer) << 24) ^
       (static_cast<uint64_t>(k.swizzle) << 8) ^ static_cast<uint64_t>(k.dtype) ^
       static_cast<uint64_t>(k.pitch) * 0x27D4EB2F165667C5ull;
  return static_cast<uint32_t>(h >> 40) % MAP_CACHE_SLOTS;
}

constexpr int DTYPE_U8 = 100;  // internal: one-byte elements (e4m3 operands of the 8-bit decode path)
static unsigned dtype_bytes(int dtype) { return dtype == DTYPE_U8 ? 1u : dtype == GMLP_F32 ? 4u : 2u; }

// 2-D row-major matrix [outer, inner] of 16-bit (DTYPE_U8: 8-bit, GMLP_F32: 32-bit) elements, swizzled rows of
// `swizzle_bytes` (32 / 64 / 128), out-of-bounds elements read as zero and are not
// written by stores.
static int encode_map(CUtensorMap* m, const void* base, int64_t inner, int64_t outer,
                      int64_t pitch_elems, uint32_t box_inner, uint32_t box_outer, int dtype,
                      int swizzle_bytes = 128) {
  const MapKey key{base, inner, outer, pitch_elems, box_inner, box_outer, dtype, swizzle_bytes};
  MapSlot& slot = g_map_cache[map_hash(key)];
  if (slot.used && slot.key == key) {
    *m = slot.map;
    return GMLP_OK;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * dtype_bytes(dtype)};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == DTYPE_U8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : dtype == GMLP_F32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == GMLP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUtensorMapSwizzle sw = swizzle_bytes == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                                : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                      : CU_TENSOR_MAP_SWIZZLE_128B;
  const CUresult r = g_encode(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GMLP_ERR_LAUNCH,
                "cuTensorMapEncodeTiled failed (%d) for base=%p inner=%lld outer=%lld pitch=%lld",
                static_cast<int>(r), base, static_cast<long long>(inner),
                static_cast<long long>(outer), static_cast<long long>(pitch_elems));
  slot.key = key;
  slot.map = *m;
  slot.used = true;
  return GMLP_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// One operand of C = A B^T as it lies in memory.
struct Operand {
  const void* ptr;
  int64_t mn;     // extent along M (for A) or N (for B)
  int64_t k;      // extent along the reduction
  int64_t ld;     // row pitch in elements
  bool mn_major;  // false: stored [mn, k]; true: stored [k, mn]
};

static int encode_operand(CUtensorMap* m, const Operand& o, uint32_t kmajor_box_rows, int dtype) {
  if (!o.ptr) return fail(GMLP_ERR_ARG, "NULL matrix pointer");
  if (!aligned16(o.ptr) || (o.ld * dtype_bytes(dtype)) % 16 != 0)
    return fail(GMLP_ERR_ALIGN, "matrix base %p / pitch %lld not 16-byte aligned", o.ptr,
                static_cast<long long>(o.ld));
  const uint32_t row = 128u / dtype_bytes(dtype);  // elements in one 128-byte row of a tile
  if (o.mn_major) return encode_map(m, o.ptr, o.mn, o.k, o.ld, row, BK, dtype);
  return encode_map(m, o.ptr, o.k, o.mn, o.ld, row, kmajor_box_rows, dtype);
}

// --------------------------------------------------------------- launching --
struct Epilogue {
  int act = ACT_SILU;
  void* out0 = nullptr;
  void* out1 = nullptr;
  void* out2 = nullptr;
  const void* in0 = nullptr;
  const void* in1 = nullptr;
  const void* bias0 = nullptr;
  const void* bias1 = nullptr;
  const float* row_scale = nullptr;
  int64_t ld_out = 0;
  int64_t ld_in = 0;
  DropoutParams drop = {};
  // row sums of the MN-major A operand (bias gradients), see GemmArgs
  void* asum_out[2] = {nullptr, nullptr};
  float* asum_part = nullptr;
  int* asum_cnt = nullptr;
  // push of other ranks' row blocks into their inboxes (tensor-parallel down projection), see GemmArgs
  char* push_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  long long push_parity_bytes = 0;
  const unsigned int* push_epoch = nullptr;
  int push_rows = 0, push_rank = 0, push_world = 0;
};

// Process-wide DEFAULTS of the three tuning knobs (set by gmlp_set_*). A call that
// carries its own values in gmlp_problem_t.tuning does not read them, so two modules
// (or two host threads, or a backward pass beside a forward pass) never change each
// other's grids through these.
//   pair mode   0 = choose per problem, 1 = always the single-CTA kernel, 2 = always the CTA pair
//   group_m     row tiles per raster group; 0 = built-in rule
//   sm_limit    CTAs a persistent GEMM grid may occupy; 0 = every SM
static std::atomic<int> g_pair_mode{0};
static std::atomic<int> g_group_m{0};
static std::atomic<int> g_sm_limit{0};

struct Tuning {
  int pair_mode, group_m, sm_limit;
  bool narrow_tiles;
};
// Field layout of the per-call word: see GMLP_TUNE_* in gmlp.h.
static Tuning resolve_tuning(uint32_t word) {
  Tuning t;
  t.pair_mode = static_cast<int>(word & 3u);
  t.group_m = static_cast<int>((word >> 2) & 0xFFFu);
  t.sm_limit = static_cast<int>((word >> 14) & 0xFFFu);
  t.narrow_tiles = (word & (1u << 27)) != 0;  // GMLP_TUNE_NARROW_TILES
  if (t.pair_mode == 0 || t.pair_mode == 3) t.pair_mode = g_pair_mode.load(std::memory_order_relaxed);
  if (t.group_m == 0) t.group_m = g_group_m.load(std::memory_order_relaxed);
  if (t.sm_limit == 0) t.sm_limit = g_sm_limit.load(std::memory_order_relaxed);
  return t;
}
static int64_t gemm_cta_budget(int sm_count, int sm_limit) {
  int64_t b = (sm_limit > 0 && sm_limit < sm_count) ? sm_limit : sm_count;
  return b < 2 ? 2 : b;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of
// before every launch.
template <typename K>
static int ensure_smem_attr(K kfn, size_t smem, std::atomic<uint64_t>& done) {
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (done.load(std::memory_order_acquire) & bit) return GMLP_OK;
  const cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
  if (e != cudaSuccess)
    return fail(GMLP_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  done.fetch_or(bit, std::memory_order_release);
  return GMLP_OK;
}

template <int BN, bool A_MN, bool B_MN, int EPI, typename T, bool ASUM>
static int launch_gemm_t(const DeviceInfo* dev, int dtype, int64_t M, int64_t N,
                         const Operand& a0, const Operand* a1, const Operand& b0,
                         const Operand* b1, int64_t k1, int batches, const Epilogue& ep,
                         uint32_t tuning_word, cudaStream_t stream) {
  const Tuning tune = resolve_tuning(tuning_word);
  // The CTA-pair kernel works on 256-row tiles; with a single row tile there is
  // nothing for the second CTA to do.
  const bool pair = tune.pair_mode == 2 || (tune.pair_mode == 0 && M > BM);
  // Shared memory: the operand ring, as deep as fits beside the epilogue's staging area.
  constexpr int B_ROWS_SINGLE = BN, B_ROWS_PAIR = BN / 2;  // rows of B a CTA stages per block
  constexpr int STAGES = gemm_stages<B_ROWS_SINGLE, EPI>();
  constexpr int PAIR_STAGES = gemm_stages<B_ROWS_PAIR, EPI>();
  static_assert(STAGES >= 3 && PAIR_STAGES >= 4, "operand ring too shallow");
  const uint32_t b_rows = pair ? BN / 2 : ((EPI == EPI_SWIGLU) ? BN / 2 : BN);
  CUtensorMap mA0, mA1, mB0, mB1;
  int rc;
  if ((rc = encode_operand(&mA0, a0, BM, dtype))) return rc;
  if ((rc = encode_operand(&mB0, b0, b_rows, dtype))) return rc;
  if (a1) {
    if ((rc = encode_operand(&mA1, *a1, BM, dtype))) return rc;
  } else {
    mA1 = mA0;
  }
  if (b1) {
    if ((rc = encode_operand(&mB1, *b1, b_rows, dtype))) return rc;
  } else {
    mB1 = mB0;
  }
  if (!ep.out0 || !aligned16(ep.out0) || (ep.ld_out * dtype_bytes(dtype)) % 16 != 0)
    return fail(GMLP_ERR_ALIGN, "output base / pitch not 16-byte aligned");
  // Output matrices as the epilogue's TMA stores see them: [32 rows x 64 columns] blocks
  // (128-byte rows) for the plain store, [32 x 32] (64-byte rows) for the gate/up kernel.
  // The dH epilogue stores through the load/store unit and takes no maps.
  CUtensorMap mO0 = mA0, mO1 = mA0, mO2 = mA0;
  constexpr bool F32 = sizeof(T) == 4;  // fp32 outputs leave as [32 x 32] blocks (128-byte rows) from both epilogues
  if (EPI == EPI_STORE) {
    const uint32_t bc = F32 ? 32 : 64;
    if ((rc = encode_map(&mO0, ep.out0, N, M, ep.ld_out, bc, 32, dtype, 128))) return rc;
    if (batches == 2) {
      if (!ep.out1 || !aligned16(ep.out1))
        return fail(GMLP_ERR_ALIGN, "second output base not 16-byte aligned");
      if ((rc = encode_map(&mO1, ep.out1, N, M, ep.ld_out, bc, 32, dtype, 128))) return rc;
    }
  } else if (EPI == EPI_SWIGLU) {
    const int sw = F32 ? 128 : 64;
    if ((rc = encode_map(&mO0, ep.out0, N, M, ep.ld_out, 32, 32, dtype, sw))) return rc;
    if (ep.out1) {
      if ((rc = encode_map(&mO1, ep.out1, N, M, ep.ld_out, 32, 32, dtype, sw))) return rc;
      if ((rc = encode_map(&mO2, ep.out2, N, M, ep.ld_out, 32, 32, dtype, sw))) return rc;
    }
  }
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.M = static_cast<int>(M);
  args.N = static_cast<int>(N);
  constexpr int ROW = row_elems<T>();  // reduction elements per stage
  args.kb0 = static_cast<int>((a0.k + ROW - 1) / ROW);
  args.kb1 = static_cast<int>((k1 + ROW - 1) / ROW);
  args.batches = batches;
  args.act = ep.act;
  args.idesc = F32 ? make_idesc_tf32(pair ? 2 * BM : BM, BN)
                   : make_idesc_f16(pair ? 2 * BM : BM, BN, dtype == GMLP_BF16 ? 1 : 0, A_MN, B_MN);
  args.status = dev->status_ptr;
  args.out0 = ep.out0;
  args.out1 = ep.out1;
  args.out2 = ep.out2;
  args.in0 = ep.in0;
  args.in1 = ep.in1;
  args.bias0 = ep.bias0;
  args.bias1 = ep.bias1;
  args.row_scale = ep.row_scale;
  args.ld_out = ep.ld_out;
  args.ld_in = ep.ld_in;
  args.drop = ep.drop;
  args.asum_out[0] = ep.asum_out[0];
  args.asum_out[1] = ep.asum_out[1];
  args.asum_part = ep.asum_part;
  args.asum_cnt = ep.asum_cnt;
  for (int i = 0; i < 8; ++i) args.push_base[i] = ep.push_base[i];
  args.push_parity_bytes = ep.push_parity_bytes;
  args.push_epoch = ep.push_epoch;
  args.push_rows = ep.push_rows;
  args.push_rank = ep.push_rank;
  args.push_world = ep.push_world;

  // Wide tiles (256 x 512 per CTA pair, one accumulator buffer): a quarter fewer operand bytes per flop, no overlap
  // of a tile's epilogue with the next main loop. For plain-store GEMMs whose reduction is long.
  constexpr bool WIDE_OK = EPI == EPI_STORE && sizeof(T) == 2 && BN == 256;
  bool wide = false;
  // (not for the pushing epilogue: its peer stores take longer than a TMA store and want the next tile's main
  // loop to hide behind)
  if (WIDE_OK && pair && !tune.narrow_tiles && ep.push_world == 0 && (args.kb0 + args.kb1) >= 32 && N >= 2 * BN) {
    // Taken when it shortens the schedule: a wide tile costs about 1.76 narrow ones (a quarter fewer operand
    // bytes, no overlap of its epilogue), and the tiles run in waves of one per CTA pair.
    const int64_t pairs = gemm_cta_budget(dev->sm_count, tune.sm_limit) / 2;
    const int64_t mt = (M + 2 * BM - 1) / (2 * BM);
    const int64_t narrow_tiles = mt * ((N + BN - 1) / BN) * batches, wide_tiles = mt * ((N + 2 * BN - 1) / (2 * BN)) * batches;
    const int64_t narrow_waves = (narrow_tiles + pairs - 1) / pairs, wide_waves = (wide_tiles + pairs - 1) / pairs;
    wide = pairs > 0 && 176 * wide_waves < 98 * narrow_waves;
  }
  const int64_t TILE_N = (EPI == EPI_SWIGLU) ? BN / 2 : (wide ? 2 * BN : BN);
  const int64_t tile_m = pair ? 2 * BM : BM;
  const int64_t m_tiles = (M + tile_m - 1) / tile_m;
  const int64_t n_tiles = (N + TILE_N - 1) / TILE_N;
  const int64_t tiles = m_tiles * n_tiles * batches;
  if (tiles <= 0 || tiles > 0x7fffffffLL) return fail(GMLP_ERR_SHAPE, "tile count out of range");
  // Raster groups: a group of row tiles sweeps all column tiles, so the tiles in
  // flight at any time (one per SM or SM pair) share a small set of A and B tiles
  // in L2, and the group's rows of A stay resident while B streams past once per group.
  // The gate/up kernel's A panel (x) is small enough to stay resident for 16 row tiles (4096
  // rows) while its wide B streams past once per group; the other kernels' panels are not,
  // and a squarer wave of tiles (8 row tiles x about 9 column tiles on 74 SM pairs) moves
  // fewer bytes.
  args.group_m = tune.group_m > 0 ? tune.group_m : (pair ? (EPI == EPI_SWIGLU ? 16 : 8) : 32);
  cudaError_t e;
  if (pair && wide) {
    if constexpr (WIDE_OK) {
      const int64_t max_pairs = gemm_cta_budget(dev->sm_count, tune.sm_limit) / 2;
      const int grid = 2 * static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
      constexpr int WIDE_STAGES = gemm_stages<2 * B_ROWS_PAIR, EPI>();
      static_assert(WIDE_STAGES >= 3, "operand ring too shallow");
      constexpr size_t smem = gemm_smem_bytes<2 * B_ROWS_PAIR, EPI, WIDE_STAGES>();
      static_assert(smem + 512 <= SMEM_LIMIT, "wide pair kernel exceeds the shared memory of an SM");
      auto kfn = gemm_tcgen05_pair_kernel<BN, A_MN, B_MN, EPI, T, WIDE_STAGES, ASUM, 2>;
      static std::atomic<uint64_t> attr_done{0};
      if ((rc = ensure_smem_attr(kfn, smem, attr_done))) return rc;
      kfn<<<grid, GEMM_THREADS, smem, stream>>>(mA0, mA1, mB0, mB1, mO0, mO1, mO2, args);
    }
  } else if (pair) {
    const int64_t max_pairs = gemm_cta_budget(dev->sm_count, tune.sm_limit) / 2;
    const int grid = 2 * static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    constexpr size_t smem = gemm_smem_bytes<B_ROWS_PAIR, EPI, PAIR_STAGES>();
    static_assert(smem + 512 <= SMEM_LIMIT, "pair kernel exceeds the shared memory of an SM");
    auto kfn = gemm_tcgen05_pair_kernel<BN, A_MN, B_MN, EPI, T, PAIR_STAGES, ASUM>;
    static std::atomic<uint64_t> attr_done{0};
    if ((rc = ensure_smem_attr(kfn, smem, attr_done))) return rc;
    kfn<<<grid, GEMM_THREADS, smem, stream>>>(mA0, mA1, mB0, mB1, mO0, mO1, mO2, args);
  } else {
    const int64_t budget = gemm_cta_budget(dev->sm_count, tune.sm_limit);
    const int grid = static_cast<int>(tiles < budget ? tiles : budget);
    constexpr size_t smem = gemm_smem_bytes<B_ROWS_SINGLE, EPI, STAGES>();
    static_assert(smem + 512 <= SMEM_LIMIT, "kernel exceeds the shared memory of an SM");
    auto kfn = gemm_tcgen05_kernel<BN, A_MN, B_MN, EPI, T, STAGES, ASUM>;
    static std::atomic<uint64_t> attr_done{0};
    if ((rc = ensure_smem_attr(kfn, smem, attr_done))) return rc;
    kfn<<<grid, GEMM_THREADS, smem, stream>>>(mA0, mA1, mB0, mB1, mO0, mO1, mO2, args);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool ASUM = false>
static int launch_gemm(const DeviceInfo* dev, int dtype, int64_t M, int64_t N, const Operand& a0,
                       const Operand* a1, const Operand& b0, const Operand* b1, int64_t k1,
                       int batches, const Epilogue& ep, uint32_t tuning_word, cudaStream_t stream) {
  if (dtype == GMLP_F32) {
    // fp32 matrices, tf32 products: K-major operands with the store and gate/up epilogues
    if constexpr (!A_MN && !B_MN && EPI != EPI_DHIDDEN && !ASUM)
      return launch_gemm_t<BN, A_MN, B_MN, EPI, float, false>(dev, dtype, M, N, a0, a1, b0, b1, k1, batches, ep,
                                                              tuning_word, stream);
    else
      return fail(GMLP_ERR_DTYPE, "fp32 matrices are supported by the forward kernels and the K-major GEMM only");
  }
  if (dtype == GMLP_BF16)
    return launch_gemm_t<BN, A_MN, B_MN, EPI, __nv_bfloat16, ASUM>(dev, dtype, M, N, a0, a1, b0, b1, k1,
                                                                   batches, ep, tuning_word, stream);
  return launch_gemm_t<BN, A_MN, B_MN, EPI, __half, ASUM>(dev, dtype, M, N, a0, a1, b0, b1, k1, batches,
                                                          ep, tuning_word, stream);
}

static int check_problem(const gmlp_problem_t* p) {
  if (!p) return fail(GMLP_ERR_ARG, "NULL problem descriptor");
  if (p->dtype != GMLP_BF16 && p->dtype != GMLP_FP16 && p->dtype != GMLP_F32)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not a gmlp_dtype_t", p->dtype);
  if (p->M <= 0 || p->K <= 0 || p->N <= 0)
    return fail(GMLP_ERR_SHAPE, "M=%lld K=%lld N=%lld must be positive",
                static_cast<long long>(p->M), static_cast<long long>(p->K),
                static_cast<long long>(p->N));
  if (p->M > 0x7fffffffLL || p->K > 0x7fffffffLL || p->N > 0x3fffffffLL)
    return fail(GMLP_ERR_SHAPE, "dimension exceeds 32-bit tile coordinates");
  if ((p->K % 8) != 0 || (p->N % 8) != 0)
    return fail(GMLP_ERR_SHAPE, "K=%lld and N=%lld must be multiples of 8",
                static_cast<long long>(p->K), static_cast<long long>(p->N));
  if (p->act < ACT_SILU || p->act > ACT_LEAKY_RELU)
    return fail(GMLP_ERR_ARG, "act=%d is not a gmlp_act_t value", p->act);
  if (!(p->dropout_p >= 0.0f && p->dropout_p < 1.0f))
    return fail(GMLP_ERR_ARG, "dropout_p=%f outside [0, 1)", static_cast<double>(p->dropout_p));
  const int64_t ng = p->N_global ? p->N_global : p->N;
  if (p->dropout_p > 0.0f && ((ng % 8) != 0 || (p->col0_global % 8) != 0 || p->row0_global < 0 ||
                              p->col0_global < 0 || p->col0_global + p->N > ng))
    return fail(GMLP_ERR_SHAPE, "dropout needs N_global and col0_global multiples of 8 and the "
                                "local columns inside [0, N_global)");
  return GMLP_OK;
}

static DropoutParams make_dropout(const gmlp_problem_t* p) {
  DropoutParams d;
  memset(&d, 0, sizeof(d));
  d.scale = 1.0f;
  d.row0_global = p->row0_global;
  d.col0_global = p->col0_global;
  d.ncols_global = p->N_global ? p->N_global : p->N;
  if (p->dropout_p > 0.0f) {
    // floor(p * 2^16), evaluated in double so the CPU restatement agrees bit for bit.
    double t = static_cast<double>(p->dropout_p) * 65536.0;
    if (t > 65535.0) t = 65535.0;
    d.thresh = static_cast<uint32_t>(t);
    d.scale = 1.0f / (1.0f - p->dropout_p);
    d.seed_lo = static_cast<uint32_t>(p->seed);
    d.seed_hi = static_cast<uint32_t>(p->seed >> 32);
    d.off_lo = static_cast<uint32_t>(p->offset);
    d.off_hi = static_cast<uint32_t>(p->offset >> 32);
  }
  return d;
}

static int check_ptrs(std::initializer_list<const void*> ps) {
  for (const void* q : ps) {
    if (!q) return fail(GMLP_ERR_ARG, "NULL pointer argument");
    if (!aligned16(q)) return fail(GMLP_ERR_ALIGN, "pointer %p is not 16-byte aligned", q);
  }
  return GMLP_OK;
}

}  // namespace gmlp

using namespace gmlp;

static int bwd_dx_impl(const gmlp_problem_t* p, const void* d_gate, const void* d_up, const void* w_gate,
                       const void* w_up, void* dx, const Epilogue* push, void* stream);

// Fills the push fields of an epilogue: output [M, K], rows owned by the ranks in shares of M / world.
static int make_push(Epilogue* ep, const gmlp_problem_t* p, int64_t max_elems, void* const* regions, int32_t rank,
                     int32_t world) {
  using namespace gmlp;
  if (!p) return fail(GMLP_ERR_ARG, "NULL problem descriptor");
  if (p->dtype != GMLP_BF16 && p->dtype != GMLP_FP16)
    return fail(GMLP_ERR_DTYPE, "the pushing epilogue takes bf16 or fp16");
  if (world < 2 || world > PEER_MAX_WORLD || rank < 0 || rank >= world)
    return fail(GMLP_ERR_ARG, "needs 2 <= world <= %d and 0 <= rank < world; got rank %d of %d", PEER_MAX_WORLD,
                rank, world);
  if (!regions) return fail(GMLP_ERR_ARG, "NULL regions");
  if (p->M <= 0 || (p->M % (32ll * world)) != 0)
    return fail(GMLP_ERR_SHAPE, "M=%lld must be a positive multiple of 32 * world so that every 32-row block has "
                                "one owner", static_cast<long long>(p->M));
  if (p->M * p->K > max_elems)
    return fail(GMLP_ERR_SHAPE, "M * K = %lld exceeds the regions' capacity of %lld elements",
                static_cast<long long>(p->M * p->K), static_cast<long long>(max_elems));
  const long long slot = peer_slot_bytes(max_elems);
  for (int r = 0; r < world; ++r) {
    if (!regions[r] || !aligned16(regions[r])) return fail(GMLP_ERR_ARG, "region of rank %d is NULL or misaligned", r);
    ep->push_base[r] = static_cast<char*>(regions[r]) + static_cast<long long>(rank) * slot;
  }
  ep->push_parity_bytes = static_cast<long long>(world) * slot;
  ep->push_epoch = reinterpret_cast<const unsigned int*>(static_cast<char*>(regions[rank]) +
                                                         peer_epoch_offset(max_elems, world));
  ep->push_rows = static_cast<int>(p->M / world);
  ep->push_rank = rank;
  ep->push_world = world;
  return GMLP_OK;
}

// The down projection, optionally with the push of other ranks' row blocks (tensor parallel).
static int down_fwd_impl(const gmlp_problem_t* p, const void* h, const void* w_down, const void* b_down,
                         const void* residual, void* y, const Epilogue* push, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({h, w_down, y}))) return rc;
  if ((b_down && !aligned16(b_down)) || (residual && !aligned16(residual)))
    return fail(GMLP_ERR_ALIGN, "bias / residual must be 16-byte aligned");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const Operand a{h, p->M, p->N, p->N, false};
  const Operand b{w_down, p->K, p->N, p->N, false};
  Epilogue ep;
  if (push) ep = *push;
  ep.out0 = y;
  ep.in0 = residual;
  ep.bias0 = b_down;
  ep.ld_out = p->K;
  ep.ld_in = p->K;
  return launch_gemm<256, false, false, EPI_STORE>(dev, p->dtype, p->M, p->K, a, nullptr, b,
                                                   nullptr, 0, 1, ep, p->tuning,
                                                   static_cast<cudaStream_t>(stream));
}

extern "C" {

int gmlp_version(void) { return 200; }

int gmlp_set_cta_pair_mode(int mode) {
  const int prev = g_pair_mode.load();
  if (mode >= 0 && mode <= 2) g_pair_mode.store(mode);
  return prev;
}

int gmlp_set_sm_limit(int sms) {
  const int prev = g_sm_limit.load();
  if (sms >= 0 && sms <= 4095) g_sm_limit.store(sms);
  return prev;
}

int gmlp_set_raster_group(int row_tiles) {
  const int prev = g_group_m.load();
  if (row_tiles >= 0 && row_tiles <= 4095) g_group_m.store(row_tiles);
  return prev;
}

const char* gmlp_last_error(void) { return g_err; }

int gmlp_status_read(int* value) {
  if (!value) return fail(GMLP_ERR_ARG, "NULL value pointer");
  const DeviceInfo* dev;
  int rc = device_info(&dev);
  if (rc) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess)
    return fail(GMLP_ERR_LAUNCH, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  int v = 0;
  e = cudaMemcpy(&v, dev->status_ptr, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaMemcpy: %s", cudaGetErrorString(e));
  if (v != 0) {
    e = cudaMemset(dev->status_ptr, 0, sizeof(int));
    if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaMemset: %s", cudaGetErrorString(e));
  }
  *value = v;
  return GMLP_OK;
}

int gmlp_hidden_fwd_scaled(const gmlp_problem_t* p, const void* x, const float* row_scale,
                           const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                           void* h, void* g_save, void* u_save, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({x, w_gate, w_up, h}))) return rc;
  if ((g_save == nullptr) != (u_save == nullptr))
    return fail(GMLP_ERR_ARG, "g_save and u_save must both be given or both be NULL");
  if ((b_gate && !aligned16(b_gate)) || (b_up && !aligned16(b_up)) ||
      (g_save && (!aligned16(g_save) || !aligned16(u_save))))
    return fail(GMLP_ERR_ALIGN, "bias / save buffers must be 16-byte aligned");
  if (row_scale && (reinterpret_cast<uintptr_t>(row_scale) & 3u) != 0)
    return fail(GMLP_ERR_ALIGN, "row_scale must be 4-byte aligned");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const Operand a{x, p->M, p->K, p->K, false};
  const Operand bg{w_gate, p->N, p->K, p->K, false};
  const Operand bu{w_up, p->N, p->K, p->K, false};
  Epilogue ep;
  ep.out0 = h;
  ep.out1 = g_save;
  ep.out2 = u_save;
  ep.bias0 = b_gate;
  ep.bias1 = b_up;
  ep.row_scale = row_scale;
  ep.ld_out = p->N;
  ep.drop = make_dropout(p);
  ep.act = p->act;
  return launch_gemm<256, false, false, EPI_SWIGLU>(dev, p->dtype, p->M, p->N, a, nullptr, bg, &bu,
                                                    0, 1, ep, p->tuning, static_cast<cudaStream_t>(stream));
}

int gmlp_hidden_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate,
                    const void* b_gate, const void* w_up, const void* b_up, void* h,
                    void* g_save, void* u_save, void* stream) {
  return gmlp_hidden_fwd_scaled(p, x, nullptr, w_gate, b_gate, w_up, b_up, h, g_save, u_save, stream);
}

int gmlp_rms_rowscale(int64_t M, int64_t K, int32_t dtype, const void* x, int64_t ld, float eps,
                      float* rs, void* xn, void* stream) {
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not GMLP_BF16 / GMLP_FP16", dtype);
  if (M <= 0 || K <= 0 || (K % 8) != 0 || (ld % 8) != 0 || ld < K)
    return fail(GMLP_ERR_SHAPE, "rms_rowscale needs M > 0, K and ld multiples of 8, ld >= K");
  if (!(eps >= 0.0f)) return fail(GMLP_ERR_ARG, "eps must be >= 0");
  if (!x || !rs) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(x) || (xn && !aligned16(xn))) return fail(GMLP_ERR_ALIGN, "x / xn must be 16-byte aligned");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  const unsigned blocks = static_cast<unsigned>((M + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == GMLP_BF16)
    rms_rowscale_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), M, K, ld, eps, rs,
                                                               static_cast<__nv_bfloat16*>(xn));
  else
    rms_rowscale_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(x), M, K, ld, eps, rs,
                                                        static_cast<__half*>(xn));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

int gmlp_rms_bwd(int64_t M, int64_t K, int32_t dtype, const void* dxn, const void* xn, const float* rs,
                 void* dx, void* stream) {
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not GMLP_BF16 / GMLP_FP16", dtype);
  if (M <= 0 || K <= 0 || (K % 8) != 0) return fail(GMLP_ERR_SHAPE, "rms_bwd needs M > 0 and K a multiple of 8");
  if (!dxn || !xn || !rs || !dx) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(dxn) || !aligned16(xn) || !aligned16(dx))
    return fail(GMLP_ERR_ALIGN, "dxn / xn / dx must be 16-byte aligned");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  const unsigned blocks = static_cast<unsigned>((M + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == GMLP_BF16)
    rms_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dxn),
                                                          static_cast<const __nv_bfloat16*>(xn), rs, M, K,
                                                          static_cast<__nv_bfloat16*>(dx));
  else
    rms_bwd_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(dxn), static_cast<const __half*>(xn),
                                                   rs, M, K, static_cast<__half*>(dx));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

int gmlp_down_fwd(const gmlp_problem_t* p, const void* h, const void* w_down,
                  const void* b_down, const void* residual, void* y, void* stream) {
  return down_fwd_impl(p, h, w_down, b_down, residual, y, nullptr, stream);
}

int gmlp_down_fwd_push(const gmlp_problem_t* p, const void* h, const void* w_down, const void* b_down,
                       const void* residual, void* y, int64_t max_elems, void* const* regions, int32_t rank,
                       int32_t world, void* stream) {
  Epilogue push;
  int rc;
  if ((rc = make_push(&push, p, max_elems, regions, rank, world))) return rc;
  return down_fwd_impl(p, h, w_down, b_down, residual, y, &push, stream);
}

int gmlp_bwd_dhidden(const gmlp_problem_t* p, const void* dy, const void* w_down,
                     const void* g, const void* u, void* d_gate, void* d_up, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({dy, w_down, g, u, d_gate, d_up}))) return rc;
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  // dH[M,N] = dy[M,K] . W_down[K,N]: the reduction runs over W_down's rows.
  const Operand a{dy, p->M, p->K, p->K, false};
  const Operand b{w_down, p->N, p->K, p->N, true};
  Epilogue ep;
  ep.out0 = d_gate;
  ep.out1 = d_up;
  ep.in0 = g;
  ep.in1 = u;
  ep.ld_out = p->N;
  ep.ld_in = p->N;
  ep.drop = make_dropout(p);
  ep.act = p->act;
  return launch_gemm<256, false, true, EPI_DHIDDEN>(dev, p->dtype, p->M, p->N, a, nullptr, b,
                                                    nullptr, 0, 1, ep, p->tuning,
                                                    static_cast<cudaStream_t>(stream));
}

int gmlp_bwd_dx(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                const void* w_gate, const void* w_up, void* dx, void* stream) {
  return bwd_dx_impl(p, d_gate, d_up, w_gate, w_up, dx, nullptr, stream);
}

int gmlp_bwd_dx_push(const gmlp_problem_t* p, const void* d_gate, const void* d_up, const void* w_gate,
                     const void* w_up, void* dx, int64_t max_elems, void* const* regions, int32_t rank,
                     int32_t world, void* stream) {
  Epilogue push;
  int rc;
  if ((rc = make_push(&push, p, max_elems, regions, rank, world))) return rc;
  return bwd_dx_impl(p, d_gate, d_up, w_gate, w_up, dx, &push, stream);
}

}  // extern "C"

static int bwd_dx_impl(const gmlp_problem_t* p, const void* d_gate, const void* d_up, const void* w_gate,
                       const void* w_up, void* dx, const Epilogue* push, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({d_gate, d_up, w_gate, w_up, dx}))) return rc;
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  // dx[M,K] = d_gate[M,N] . W_gate[N,K] + d_up[M,N] . W_up[N,K]: one accumulator,
  // two reduction segments of length N.
  const Operand a0{d_gate, p->M, p->N, p->N, false};
  const Operand a1{d_up, p->M, p->N, p->N, false};
  const Operand b0{w_gate, p->K, p->N, p->K, true};
  const Operand b1{w_up, p->K, p->N, p->K, true};
  Epilogue ep;
  if (push) ep = *push;
  ep.out0 = dx;
  ep.ld_out = p->K;
  return launch_gemm<256, false, true, EPI_STORE>(dev, p->dtype, p->M, p->K, a0, &a1, b0, &b1,
                                                  p->N, 1, ep, p->tuning,
                                                  static_cast<cudaStream_t>(stream));
}

extern "C" {

// Scratch of the fused bias-gradient sums for an output of `mn` rows whose GEMM has `cols`
// output columns and `batches` problems: arrival counters (one per 128 rows and batch;
// must be zero) followed by the fp32 partial sums [batches][column tiles][rows padded to 256].
struct AsumLayout {
  size_t cnt_bytes, part_bytes;
};
static AsumLayout asum_layout(int64_t mn, int64_t cols, int batches) {
  const int64_t mn_pad = (mn + 255) / 256 * 256, n_tiles = (cols + 255) / 256;
  AsumLayout l;
  l.cnt_bytes = (static_cast<size_t>(batches) * (mn_pad / 128) * sizeof(int) + 255) / 256 * 256;
  l.part_bytes = static_cast<size_t>(batches) * n_tiles * mn_pad * sizeof(float);
  return l;
}

// The two weight-gradient kernels of a module share one scratch buffer, one after the other: their arrival
// counters (which each kernel leaves at zero) sit in a common region at the front, sized for the larger of
// the two, and the fp32 partial sums (scratch proper) behind it, so that neither kernel's partial sums can
// ever land on the other's counters.
static size_t asum_common_cnt_bytes(const gmlp_problem_t* p) {
  return std::max(asum_layout(p->N, p->K, 2).cnt_bytes, asum_layout(p->K, p->N, 1).cnt_bytes);
}

static int dw_gate_up_impl(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                           const void* x, void* dw_gate, void* dw_up, void* db_gate, void* db_up,
                           void* scratch, size_t scratch_bytes, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({d_gate, d_up, x, dw_gate, dw_up}))) return rc;
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  // dW[N,K] = d^T[N,M] . x[M,K]: both operands lie token-major, the reduction
  // runs over their rows. Two problems share x.
  const Operand a0{d_gate, p->N, p->M, p->N, true};
  const Operand a1{d_up, p->N, p->M, p->N, true};
  const Operand b{x, p->K, p->M, p->K, true};
  Epilogue ep;
  ep.out0 = dw_gate;
  ep.out1 = dw_up;
  ep.ld_out = p->K;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!db_gate && !db_up)
    return launch_gemm<256, true, true, EPI_STORE>(dev, p->dtype, p->N, p->K, a0, &a1, b, nullptr, 0,
                                                   2, ep, p->tuning, st);
  // db[n] = sum over tokens of d[token, n]: the row sums of this GEMM's A operand
  if ((db_gate && !aligned16(db_gate)) || (db_up && !aligned16(db_up)))
    return fail(GMLP_ERR_ALIGN, "bias gradient buffers must be 16-byte aligned");
  const AsumLayout l = asum_layout(p->N, p->K, 2);
  const size_t cnt_bytes = asum_common_cnt_bytes(p);
  if (!scratch || !aligned16(scratch) || scratch_bytes < cnt_bytes + l.part_bytes)
    return fail(GMLP_ERR_SCRATCH, "bias-gradient scratch holds %zu bytes, %zu needed", scratch_bytes,
                cnt_bytes + l.part_bytes);
  ep.asum_out[0] = db_gate;
  ep.asum_out[1] = db_up;
  ep.asum_cnt = static_cast<int*>(scratch);
  ep.asum_part = reinterpret_cast<float*>(static_cast<char*>(scratch) + cnt_bytes);
  return launch_gemm<256, true, true, EPI_STORE, true>(dev, p->dtype, p->N, p->K, a0, &a1, b, nullptr,
                                                       0, 2, ep, p->tuning, st);
}

static int dw_down_impl(const gmlp_problem_t* p, const void* dy, const void* h, void* dw_down,
                        void* db_down, void* scratch, size_t scratch_bytes, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({dy, h, dw_down}))) return rc;
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  // dW_down[K,N] = dy^T[K,M] . h[M,N]
  const Operand a{dy, p->K, p->M, p->K, true};
  const Operand b{h, p->N, p->M, p->N, true};
  Epilogue ep;
  ep.out0 = dw_down;
  ep.ld_out = p->N;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!db_down)
    return launch_gemm<256, true, true, EPI_STORE>(dev, p->dtype, p->K, p->N, a, nullptr, b, nullptr,
                                                   0, 1, ep, p->tuning, st);
  if (!aligned16(db_down)) return fail(GMLP_ERR_ALIGN, "bias gradient buffer must be 16-byte aligned");
  const AsumLayout l = asum_layout(p->K, p->N, 1);
  const size_t cnt_bytes = asum_common_cnt_bytes(p);
  if (!scratch || !aligned16(scratch) || scratch_bytes < cnt_bytes + l.part_bytes)
    return fail(GMLP_ERR_SCRATCH, "bias-gradient scratch holds %zu bytes, %zu needed", scratch_bytes,
                cnt_bytes + l.part_bytes);
  ep.asum_out[0] = db_down;
  ep.asum_cnt = static_cast<int*>(scratch);
  ep.asum_part = reinterpret_cast<float*>(static_cast<char*>(scratch) + cnt_bytes);
  return launch_gemm<256, true, true, EPI_STORE, true>(dev, p->dtype, p->K, p->N, a, nullptr, b,
                                                       nullptr, 0, 1, ep, p->tuning, st);
}

int gmlp_bwd_dw_gate_up(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                        const void* x, void* dw_gate, void* dw_up, void* stream) {
  return dw_gate_up_impl(p, d_gate, d_up, x, dw_gate, dw_up, nullptr, nullptr, nullptr, 0, stream);
}

int gmlp_bwd_dw_down(const gmlp_problem_t* p, const void* dy, const void* h, void* dw_down,
                     void* stream) {
  return dw_down_impl(p, dy, h, dw_down, nullptr, nullptr, 0, stream);
}

size_t gmlp_bias_grad_scratch_bytes(const gmlp_problem_t* p) {
  if (!p || p->K <= 0 || p->N <= 0) return 0;
  const AsumLayout a = asum_layout(p->N, p->K, 2), b = asum_layout(p->K, p->N, 1);
  return asum_common_cnt_bytes(p) + std::max(a.part_bytes, b.part_bytes);
}

int gmlp_bwd_dw_gate_up_bias(const gmlp_problem_t* p, const void* d_gate, const void* d_up,
                             const void* x, void* dw_gate, void* dw_up, void* db_gate, void* db_up,
                             void* scratch, size_t scratch_bytes, void* stream) {
  return dw_gate_up_impl(p, d_gate, d_up, x, dw_gate, dw_up, db_gate, db_up, scratch, scratch_bytes,
                         stream);
}

int gmlp_bwd_dw_down_bias(const gmlp_problem_t* p, const void* dy, const void* h, void* dw_down,
                          void* db_down, void* scratch, size_t scratch_bytes, void* stream) {
  return dw_down_impl(p, dy, h, dw_down, db_down, scratch, scratch_bytes, stream);
}

int gmlp_mlp_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate, const void* b_gate,
                 const void* w_up, const void* b_up, const void* w_down, const void* b_down,
                 const void* residual, void* h, void* g_save, void* u_save, void* y, void* stream) {
  int rc;
  if ((rc = gmlp_hidden_fwd(p, x, w_gate, b_gate, w_up, b_up, h, g_save, u_save, stream))) return rc;
  return gmlp_down_fwd(p, h, w_down, b_down, residual, y, stream);
}

int gmlp_mlp_bwd(const gmlp_problem_t* p, const void* dy, const void* x, const void* w_gate,
                 const void* w_up, const void* w_down, const void* g, const void* u, const void* h,
                 void* d_gate, void* d_up, void* dx, void* dw_gate, void* dw_up, void* dw_down,
                 void* db_gate, void* db_up, void* db_down, void* scratch, size_t scratch_bytes,
                 void* stream) {
  int rc;
  if ((dw_gate == nullptr) != (dw_up == nullptr))
    return fail(GMLP_ERR_ARG, "dw_gate and dw_up must both be given or both be NULL");
  if ((db_gate || db_up) && !dw_gate)
    return fail(GMLP_ERR_ARG, "db_gate / db_up are taken inside the dW_gate / dW_up GEMM: pass dw_gate and "
                              "dw_up as well, or use gmlp_colsum");
  if (db_down && !dw_down)
    return fail(GMLP_ERR_ARG, "db_down is taken inside the dW_down GEMM: pass dw_down as well, or use "
                              "gmlp_colsum");
  const bool hidden = dx || dw_gate;
  if (hidden) {
    if (!d_gate || !d_up) return fail(GMLP_ERR_ARG, "d_gate and d_up buffers are needed for dx / dW_gate / dW_up");
    if ((rc = gmlp_bwd_dhidden(p, dy, w_down, g, u, d_gate, d_up, stream))) return rc;
    if (dx && (rc = gmlp_bwd_dx(p, d_gate, d_up, w_gate, w_up, dx, stream))) return rc;
    if (dw_gate && (rc = gmlp_bwd_dw_gate_up_bias(p, d_gate, d_up, x, dw_gate, dw_up, db_gate, db_up, scratch,
                                                  scratch_bytes, stream)))
      return rc;
  }
  if (dw_down && (rc = gmlp_bwd_dw_down_bias(p, dy, h, dw_down, db_down, scratch, scratch_bytes, stream)))
    return rc;
  return GMLP_OK;
}

int gmlp_bwd_dact(const gmlp_problem_t* p, const void* dh, const void* g, const void* u,
                  void* d_gate, void* d_up, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if ((rc = check_ptrs({dh, g, u, d_gate, d_up}))) return rc;
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const DropoutParams d = make_dropout(p);
  const long long groups = p->M * (p->N / 8);
  long long blocks = (groups + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->dtype == GMLP_F32)
    dact_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const float*>(dh), static_cast<const float*>(g), static_cast<const float*>(u),
        static_cast<float*>(d_gate), static_cast<float*>(d_up), p->M, p->N, d, p->act);
  else if (p->dtype == GMLP_BF16)
    dact_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dh), static_cast<const __nv_bfloat16*>(g),
        static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(d_gate),
        static_cast<__nv_bfloat16*>(d_up), p->M, p->N, d, p->act);
  else
    dact_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __half*>(dh), static_cast<const __half*>(g),
        static_cast<const __half*>(u), static_cast<__half*>(d_gate), static_cast<__half*>(d_up),
        p->M, p->N, d, p->act);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

int gmlp_dropout_mask(const gmlp_problem_t* p, uint8_t* mask, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if (!mask) return fail(GMLP_ERR_ARG, "NULL mask pointer");
  if ((reinterpret_cast<uintptr_t>(mask) & 7u) != 0)
    return fail(GMLP_ERR_ALIGN, "mask must be 8-byte aligned");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const DropoutParams d = make_dropout(p);
  const long long quads = p->M * (p->N / 8);
  long long blocks = (quads + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  dropout_mask_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, p->M, p->N, d);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

// Row blocks of the column-sum kernels. The target is a fixed number of thread blocks
// (a few per SM on any sm_100 part) rather than a multiple of the device's SM count, so
// that the scratch size is a function of the shape alone and can be computed without a
// device (gmlp_colsum_scratch_bytes takes none).
constexpr int64_t COLSUM_TARGET_BLOCKS = 592;
static int colsum_row_blocks(int64_t rows, int64_t cols) {
  const int64_t col_blocks = (cols + COLSUM_COLS - 1) / COLSUM_COLS;
  int64_t rb = (COLSUM_TARGET_BLOCKS + col_blocks - 1) / col_blocks;
  const int64_t max_rb = (rows + 63) / 64;  // at least 64 rows per block
  if (rb > max_rb) rb = max_rb;
  if (rb < 1) rb = 1;
  return static_cast<int>(rb);
}

static int colsum_check(int64_t rows, int64_t cols, int32_t dtype, const void* src, int64_t ld,
                        const void* dst) {
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16 && dtype != GMLP_F32)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not a gmlp_dtype_t", dtype);
  if (rows <= 0 || cols <= 0 || (cols % 8) != 0 || (ld % 8) != 0 || ld < cols)
    return fail(GMLP_ERR_SHAPE, "colsum needs rows > 0, cols and ld multiples of 8, ld >= cols");
  if (!src || !dst) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(src)) return fail(GMLP_ERR_ALIGN, "src must be 16-byte aligned");
  return GMLP_OK;
}

// Both passes of a column sum with the fp32 partial sums in `part` (device memory of at
// least gmlp_colsum_scratch_bytes(rows, cols) bytes, wherever it comes from). Pass 1
// writes every partial sum that pass 2 reads, so `part` needs no clearing.
static int colsum_launch(int64_t rows, int64_t cols, int32_t dtype, const void* src, int64_t ld,
                         float* part, void* dst, cudaStream_t st) {
  const int rb = colsum_row_blocks(rows, cols);
  const long long rows_per_block = (rows + rb - 1) / rb;
  const dim3 grid(static_cast<unsigned>((cols + COLSUM_COLS - 1) / COLSUM_COLS),
                  static_cast<unsigned>(rb));
  const unsigned fin_blocks = static_cast<unsigned>((cols + 255) / 256);
  if (dtype == GMLP_F32) {
    colsum_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), rows, cols, ld,
                                                       rows_per_block, part);
    colsum_final_kernel<float><<<fin_blocks, 256, 0, st>>>(part, cols, rb, static_cast<float*>(dst));
  } else if (dtype == GMLP_BF16) {
    colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(src), rows, cols, ld, rows_per_block, part);
    colsum_final_kernel<__nv_bfloat16><<<fin_blocks, 256, 0, st>>>(
        part, cols, rb, static_cast<__nv_bfloat16*>(dst));
  } else {
    colsum_partial_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(src), rows,
                                                        cols, ld, rows_per_block, part);
    colsum_final_kernel<__half><<<fin_blocks, 256, 0, st>>>(part, cols, rb,
                                                            static_cast<__half*>(dst));
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

size_t gmlp_colsum_scratch_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>(colsum_row_blocks(rows, cols)) * static_cast<size_t>(cols) *
         sizeof(float);
}

int gmlp_colsum(int64_t rows, int64_t cols, int32_t dtype, const void* src, int64_t ld,
                void* scratch, size_t scratch_bytes, void* dst, void* stream) {
  int rc;
  if ((rc = colsum_check(rows, cols, dtype, src, ld, dst))) return rc;
  if (!scratch) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(scratch)) return fail(GMLP_ERR_ALIGN, "scratch must be 16-byte aligned");
  if (scratch_bytes < gmlp_colsum_scratch_bytes(rows, cols))
    return fail(GMLP_ERR_SCRATCH, "scratch holds %zu bytes, %zu needed", scratch_bytes,
                gmlp_colsum_scratch_bytes(rows, cols));
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  return colsum_launch(rows, cols, dtype, src, ld, static_cast<float*>(scratch), dst,
                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ------------------------------------------------------------------ decode --
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct DecodeLayout {
  int mpad;
  size_t counters1_off, counters2_off, sync_off, slots_off, total;
};
static DecodeLayout decode_layout(const gmlp_problem_t* p, int ctas) {
  DecodeLayout l;
  l.mpad = p->M <= 16 ? 16 : (p->M <= 32 ? 32 : 64);
  const size_t t1 = static_cast<size_t>((p->N + 127) / 128), t2 = static_cast<size_t>((p->K + 127) / 128);
  l.counters1_off = 0;
  l.counters2_off = align_up(t1 * sizeof(int), 256);
  l.sync_off = l.counters2_off + align_up(t2 * sizeof(int), 256);  // the one-launch kernel's two device-wide counts
  l.slots_off = l.sync_off + 256;
  // one slot holds a CTA's partial row tile: all sub-tiles and accumulators of the larger kernel
  const size_t accs = l.mpad == 16
                          ? std::max<size_t>(2 * decode_subtiles<16, true>(), decode_subtiles<16, false>())
                          : l.mpad == 32
                                ? std::max<size_t>(2 * decode_subtiles<32, true>(), decode_subtiles<32, false>())
                                : std::max<size_t>(2 * decode_subtiles<64, true>(), decode_subtiles<64, false>());
  l.total = l.slots_off + 2ull * ctas * accs * 128ull * l.mpad * sizeof(float);
  return l;
}

// Per-weight-row dequantisation scales of the 8-bit path (null on the 16-bit path).
struct WeightScales {
  const float* s0 = nullptr;
  const float* s1 = nullptr;
};

template <int MPAD, bool DUAL, typename T, bool FP8>
static int launch_decode_t(const DeviceInfo* dev, int dtype, int M, int64_t rows, int64_t red,
                           const void* w0, const void* w1, const void* act, int64_t act_ld,
                           const void* bias0, const void* bias1, const void* residual,
                           const float* row_scale, WeightScales ws, void* out, int64_t ld_out, float* slots,
                           int* counters, bool dependent, int gate_act, cudaStream_t stream) {
  CUtensorMap mW0, mW1, mAct;
  int rc;
  constexpr int BOX_ROWS = decode_box_rows<MPAD, DUAL>();
  constexpr int TILE_ROWS = 128 * decode_subtiles<MPAD, DUAL>();
  constexpr int RED = FP8 ? 128 : BK;            // reduction elements per 128-byte row
  const int op_dtype = FP8 ? DTYPE_U8 : dtype;  // element type of weights and activations
  if ((rc = encode_map(&mW0, w0, red, rows, red, RED, BOX_ROWS, op_dtype))) return rc;
  if (DUAL) {
    if ((rc = encode_map(&mW1, w1, red, rows, red, RED, BOX_ROWS, op_dtype))) return rc;
  } else {
    mW1 = mW0;
  }
  if ((rc = encode_map(&mAct, act, red, M, act_ld, RED, MPAD, op_dtype))) return rc;
  DecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.rows = static_cast<int>(rows);
  a.kbt = static_cast<int>((red + RED - 1) / RED);
  a.idesc = FP8 ? make_idesc_f8(128, MPAD) : make_idesc_f16(128, MPAD, dtype == GMLP_BF16 ? 1 : 0, false, false);
  a.wscale0 = ws.s0;
  a.wscale1 = ws.s1;
  a.status = dev->status_ptr;
  a.bias0 = bias0;
  a.bias1 = bias1;
  a.out = out;
  a.residual = residual;
  a.row_scale = row_scale;
  a.ld_out = ld_out;
  a.slots = slots;
  a.counters = counters;
  a.dependent = dependent ? 1 : 0;
  a.act = gate_act;
  const long long total = ((rows + TILE_ROWS - 1) / TILE_ROWS) * static_cast<long long>(a.kbt);
  const int grid = static_cast<int>(total < dev->sm_count ? total : dev->sm_count);
  constexpr size_t smem = decode_smem_bytes<MPAD, DUAL>();
  auto kfn = decode_stream_kernel<MPAD, DUAL, T, FP8>;
  static std::atomic<uint64_t> attr_done{0};
  if ((rc = ensure_smem_attr(kfn, smem, attr_done))) return rc;
  cudaError_t e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(DECODE_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {
    // Let this grid's CTAs start (and stream weights) while the preceding grid drains.
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  e = cudaLaunchKernelEx(&cfg, kfn, mW0, mW1, mAct, a);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

template <bool DUAL, bool FP8 = false, typename... Args>
static int launch_decode(int mpad, int dtype, Args... args) {
  const bool bf = dtype == GMLP_BF16;
  if (mpad == 16)
    return bf ? launch_decode_t<16, DUAL, __nv_bfloat16, FP8>(args...)
              : launch_decode_t<16, DUAL, __half, FP8>(args...);
  if (mpad == 32)
    return bf ? launch_decode_t<32, DUAL, __nv_bfloat16, FP8>(args...)
              : launch_decode_t<32, DUAL, __half, FP8>(args...);
  return bf ? launch_decode_t<64, DUAL, __nv_bfloat16, FP8>(args...)
            : launch_decode_t<64, DUAL, __half, FP8>(args...);
}

// Both projections from one launch (decode_fused.cuh).
template <int MPAD, typename T>
static int launch_decode_fused_t(const DeviceInfo* dev, const gmlp_problem_t* p, const void* x,
                                 const float* row_scale, const void* w_gate, const void* b_gate, const void* w_up,
                                 const void* b_up, const void* w_down, const void* b_down, const void* residual,
                                 void* h, void* y, float* slots, int* counters1, int* counters2, int* sync,
                                 bool dependent, cudaStream_t stream) {
  CUtensorMap mWg, mWu, mWd, mX, mH;
  int rc;
  const int M = static_cast<int>(p->M);
  if ((rc = encode_map(&mWg, w_gate, p->K, p->N, p->K, BK, 128, p->dtype))) return rc;
  if ((rc = encode_map(&mWu, w_up, p->K, p->N, p->K, BK, 128, p->dtype))) return rc;
  if ((rc = encode_map(&mWd, w_down, p->N, p->K, p->N, BK, 128, p->dtype))) return rc;
  if ((rc = encode_map(&mX, x, p->K, M, p->K, BK, MPAD, p->dtype))) return rc;
  if ((rc = encode_map(&mH, h, p->N, M, p->N, BK, MPAD, p->dtype))) return rc;
  DecodeFusedArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.N = static_cast<int>(p->N);
  a.K = static_cast<int>(p->K);
  a.idesc = make_idesc_f16(128, MPAD, p->dtype == GMLP_BF16 ? 1 : 0, false, false);
  a.status = dev->status_ptr;
  a.b_gate = b_gate;
  a.b_up = b_up;
  a.b_down = b_down;
  a.h = h;
  a.y = y;
  a.residual = residual;
  a.row_scale = row_scale;
  a.slots = slots;
  a.counters1 = counters1;
  a.counters2 = counters2;
  a.sync = sync;
  a.act = p->act;
  a.dependent = dependent ? 1 : 0;
  const long long total1 = ((p->N + 127) / 128) * (p->K / BK), total2 = ((p->K + 127) / 128) * (p->N / BK);
  const long long most = std::max(total1, total2);
  const int grid = static_cast<int>(most < dev->sm_count ? most : dev->sm_count);
  constexpr size_t smem = fused_smem_bytes<MPAD>();
  auto kfn = decode_fused_kernel<MPAD, T>;
  static std::atomic<uint64_t> attr_done{0};
  if ((rc = ensure_smem_attr(kfn, smem, attr_done))) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(DECODE_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, mWg, mWu, mWd, mX, mH, a);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

extern "C" {

size_t gmlp_decode_scratch_bytes(const gmlp_problem_t* p) {
  if (!p || p->M <= 0 || p->M > 64 || p->K <= 0 || p->N <= 0) return 0;
  const DeviceInfo* dev;
  int ctas = 256;  // without a device: an upper bound on the SM count
  if (device_info(&dev) == GMLP_OK) ctas = dev->sm_count;
  return decode_layout(p, ctas).total;
}

int gmlp_decode_fwd_scaled(const gmlp_problem_t* p, const void* x, const float* row_scale,
                           const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                           const void* w_down, const void* b_down, const void* residual, void* h, void* y,
                           void* scratch, size_t scratch_bytes, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if (p->M > 64) return fail(GMLP_ERR_SHAPE, "decode path takes at most 64 tokens, got %lld",
                             static_cast<long long>(p->M));
  if (p->dropout_p != 0.0f) return fail(GMLP_ERR_ARG, "decode path is inference only: dropout_p must be 0");
  if ((rc = check_ptrs({x, w_gate, w_up, w_down, h, y, scratch}))) return rc;
  if ((p->K % 64) != 0 || (p->N % 64) != 0)
    return fail(GMLP_ERR_SHAPE, "decode path needs K and N multiples of 64");
  if (row_scale && (reinterpret_cast<uintptr_t>(row_scale) & 3u) != 0)
    return fail(GMLP_ERR_ALIGN, "row_scale must be 4-byte aligned");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const DecodeLayout l = decode_layout(p, dev->sm_count);
  if (scratch_bytes < l.total)
    return fail(GMLP_ERR_SCRATCH, "scratch holds %zu bytes, %zu needed", scratch_bytes, l.total);
  char* sc = static_cast<char*>(scratch);
  float* slots = reinterpret_cast<float*>(sc + l.slots_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int M = static_cast<int>(p->M);
  // GMLP_TUNE_ORDINARY_LAUNCH: the first kernel is launched as an ordinary kernel, i.e. it starts
  // (and reads weights) only when everything before it on the stream has finished.
  const bool dep = (p->tuning & (1u << 26)) == 0;
  // H[M,N] = act(x Wg^T + bg) * (x Wu^T + bu): weight rows = N, reduction = K. Both kernels
  // are launched as programmatic dependents of whatever precedes them in the stream: they
  // start streaming weights at once and wait for the predecessor only before they read
  // activations or touch h, y or the scratch (which a preceding decode call may still use).
  rc = launch_decode<true>(l.mpad, p->dtype, dev, p->dtype, M, p->N, p->K, w_gate, w_up, x, p->K,
                           b_gate, b_up, static_cast<const void*>(nullptr), row_scale, WeightScales{}, h, p->N,
                           slots, reinterpret_cast<int*>(sc + l.counters1_off), dep, p->act, st);
  if (rc) return rc;
  // y[M,K] = h Wd^T + bd: weight rows = K, reduction = N
  return launch_decode<false>(l.mpad, p->dtype, dev, p->dtype, M, p->K, p->N, w_down,
                              static_cast<const void*>(nullptr), static_cast<const void*>(h), p->N, b_down,
                              static_cast<const void*>(nullptr), residual, static_cast<const float*>(nullptr),
                              WeightScales{}, y, p->K, slots, reinterpret_cast<int*>(sc + l.counters2_off), true,
                              p->act, st);
}

static int quantize_rows_launch(int64_t M, int64_t K, int32_t dtype, const void* x, int64_t ld, void* q,
                                float* scale, bool dependent, void* stream) {
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not GMLP_BF16 / GMLP_FP16", dtype);
  if (M <= 0 || K <= 0 || (K % 8) != 0 || (ld % 8) != 0 || ld < K || M > 0x7fffffffLL)
    return fail(GMLP_ERR_SHAPE, "quantize_rows needs M > 0, K and ld multiples of 8, ld >= K");
  if (!x || !q || !scale) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u) != 0)
    return fail(GMLP_ERR_ALIGN, "x must be 16-byte and q 8-byte aligned");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(M));
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  const int dep = dependent ? 1 : 0;
  long long m = M, k = K, l = ld;
  uint8_t* q8 = static_cast<uint8_t*>(q);
  cudaError_t e;
  if (dtype == GMLP_BF16)
    e = cudaLaunchKernelEx(&cfg, quantize_rows_e4m3_kernel<__nv_bfloat16>, static_cast<const __nv_bfloat16*>(x), m, k,
                           l, q8, scale, dep);
  else
    e = cudaLaunchKernelEx(&cfg, quantize_rows_e4m3_kernel<__half>, static_cast<const __half*>(x), m, k, l, q8, scale,
                           dep);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

int gmlp_quantize_rows_e4m3(int64_t M, int64_t K, int32_t dtype, const void* x, int64_t ld, void* q,
                            float* scale, void* stream) {
  return quantize_rows_launch(M, K, dtype, x, ld, q, scale, false, stream);
}

int gmlp_decode_fwd_fused(const gmlp_problem_t* p, const void* x, const float* row_scale,
                          const void* w_gate, const void* b_gate, const void* w_up, const void* b_up,
                          const void* w_down, const void* b_down, const void* residual, void* h, void* y,
                          void* scratch, size_t scratch_bytes, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if (p->dtype != GMLP_BF16 && p->dtype != GMLP_FP16)
    return fail(GMLP_ERR_ARG, "the one-launch decode path takes bf16 or fp16");
  if (p->M > 64) return fail(GMLP_ERR_SHAPE, "decode path takes at most 64 tokens, got %lld",
                             static_cast<long long>(p->M));
  if (p->dropout_p != 0.0f) return fail(GMLP_ERR_ARG, "decode path is inference only: dropout_p must be 0");
  if ((rc = check_ptrs({x, w_gate, w_up, w_down, h, y, scratch}))) return rc;
  if ((p->K % 64) != 0 || (p->N % 64) != 0)
    return fail(GMLP_ERR_SHAPE, "decode path needs K and N multiples of 64");
  if (row_scale && (reinterpret_cast<uintptr_t>(row_scale) & 3u) != 0)
    return fail(GMLP_ERR_ALIGN, "row_scale must be 4-byte aligned");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const DecodeLayout l = decode_layout(p, dev->sm_count);
  if (scratch_bytes < l.total)
    return fail(GMLP_ERR_SCRATCH, "scratch holds %zu bytes, %zu needed", scratch_bytes, l.total);
  char* sc = static_cast<char*>(scratch);
  float* slots = reinterpret_cast<float*>(sc + l.slots_off);
  int* c1 = reinterpret_cast<int*>(sc + l.counters1_off);
  int* c2 = reinterpret_cast<int*>(sc + l.counters2_off);
  int* sync = reinterpret_cast<int*>(sc + l.sync_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool dep = (p->tuning & (1u << 26)) == 0;  // GMLP_TUNE_ORDINARY_LAUNCH, as in gmlp_decode_fwd
  const bool bf = p->dtype == GMLP_BF16;
#define GMLP_FUSED(MP)                                                                                             \
  (bf ? launch_decode_fused_t<MP, __nv_bfloat16>(dev, p, x, row_scale, w_gate, b_gate, w_up, b_up, w_down, b_down, \
                                                 residual, h, y, slots, c1, c2, sync, dep, st)                     \
      : launch_decode_fused_t<MP, __half>(dev, p, x, row_scale, w_gate, b_gate, w_up, b_up, w_down, b_down,        \
                                          residual, h, y, slots, c1, c2, sync, dep, st))
  if (l.mpad == 16) return GMLP_FUSED(16);
  if (l.mpad == 32) return GMLP_FUSED(32);
  return GMLP_FUSED(64);
#undef GMLP_FUSED
}

int gmlp_decode_fwd_fp8(const gmlp_problem_t* p, const void* x, const void* w_gate8,
                        const float* w_gate_scale, const void* b_gate, const void* w_up8,
                        const float* w_up_scale, const void* b_up, const void* w_down8,
                        const float* w_down_scale, const void* b_down, const void* residual, void* x8,
                        float* x_scale, void* h, void* h8, float* h_scale, void* y, void* scratch,
                        size_t scratch_bytes, void* stream) {
  int rc;
  if ((rc = check_problem(p))) return rc;
  if (p->M > 64) return fail(GMLP_ERR_SHAPE, "decode path takes at most 64 tokens, got %lld",
                             static_cast<long long>(p->M));
  if (p->dropout_p != 0.0f) return fail(GMLP_ERR_ARG, "decode path is inference only: dropout_p must be 0");
  if ((rc = check_ptrs({x, w_gate8, w_up8, w_down8, x8, h, h8, y, scratch}))) return rc;
  if (!w_gate_scale || !w_up_scale || !w_down_scale || !x_scale || !h_scale)
    return fail(GMLP_ERR_ARG, "NULL scale pointer");
  if ((p->K % 128) != 0 || (p->N % 128) != 0)
    return fail(GMLP_ERR_SHAPE, "the 8-bit decode path needs K and N multiples of 128");
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  const DecodeLayout l = decode_layout(p, dev->sm_count);
  if (scratch_bytes < l.total)
    return fail(GMLP_ERR_SCRATCH, "scratch holds %zu bytes, %zu needed", scratch_bytes, l.total);
  char* sc = static_cast<char*>(scratch);
  float* slots = reinterpret_cast<float*>(sc + l.slots_off);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int M = static_cast<int>(p->M);
  // x -> e4m3 with one scale per token; gate/up kernel on 8-bit operands (accumulators times token
  // scale times weight-row scale); H (16-bit) -> e4m3 per token; down projection likewise.
  // The quantisers run as programmatic dependents too, so the kernel after each of them starts
  // streaming its weights while the one before it drains.
  const bool dep = (p->tuning & (1u << 26)) == 0;  // GMLP_TUNE_ORDINARY_LAUNCH, as in gmlp_decode_fwd
  if ((rc = quantize_rows_launch(M, p->K, p->dtype, x, p->K, x8, x_scale, dep, stream))) return rc;
  rc = launch_decode<true, true>(l.mpad, p->dtype, dev, p->dtype, M, p->N, p->K, w_gate8, w_up8,
                                 static_cast<const void*>(x8), p->K, b_gate, b_up, static_cast<const void*>(nullptr),
                                 static_cast<const float*>(x_scale), WeightScales{w_gate_scale, w_up_scale}, h, p->N,
                                 slots, reinterpret_cast<int*>(sc + l.counters1_off), dep, p->act, st);
  if (rc) return rc;
  if ((rc = quantize_rows_launch(M, p->N, p->dtype, h, p->N, h8, h_scale, true, stream))) return rc;
  return launch_decode<false, true>(l.mpad, p->dtype, dev, p->dtype, M, p->K, p->N, w_down8,
                                    static_cast<const void*>(nullptr), static_cast<const void*>(h8), p->N, b_down,
                                    static_cast<const void*>(nullptr), residual, static_cast<const float*>(h_scale),
                                    WeightScales{w_down_scale, nullptr}, y, p->K, slots,
                                    reinterpret_cast<int*>(sc + l.counters2_off), true, p->act, st);
}

int gmlp_decode_fwd(const gmlp_problem_t* p, const void* x, const void* w_gate,
                    const void* b_gate, const void* w_up, const void* b_up, const void* w_down,
                    const void* b_down, const void* residual, void* h, void* y, void* scratch,
                    size_t scratch_bytes, void* stream) {
  return gmlp_decode_fwd_scaled(p, x, nullptr, w_gate, b_gate, w_up, b_up, w_down, b_down, residual, h, y,
                                scratch, scratch_bytes, stream);
}

int gmlp_gemm(int32_t dtype, int32_t a_mn, int32_t b_mn, int64_t M, int64_t N, int64_t K,
              const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
              const void* bias, void* stream) {
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16 && dtype != GMLP_F32)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not a gmlp_dtype_t", dtype);
  if (M <= 0 || N <= 0 || K <= 0 || (N % 8) != 0 || (ldc % 8) != 0 || M > 0x7fffffffLL ||
      N > 0x7fffffffLL || K > 0x7fffffffLL)
    return fail(GMLP_ERR_SHAPE, "gemm needs positive M, N, K; N and ldc multiples of 8");
  if (!C || !aligned16(C) || (bias && !aligned16(bias)))
    return fail(GMLP_ERR_ALIGN, "C / bias must be non-NULL and 16-byte aligned");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  const Operand a{A, M, K, lda, a_mn != 0};
  const Operand b{B, N, K, ldb, b_mn != 0};
  Epilogue ep;
  ep.out0 = C;
  ep.bias0 = bias;
  ep.ld_out = ldc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn)
    return launch_gemm<256, false, false, EPI_STORE>(dev, dtype, M, N, a, nullptr, b, nullptr, 0,
                                                     1, ep, 0u, st);
  if (!a_mn && b_mn)
    return launch_gemm<256, false, true, EPI_STORE>(dev, dtype, M, N, a, nullptr, b, nullptr, 0, 1,
                                                    ep, 0u, st);
  if (a_mn && b_mn)
    return launch_gemm<256, true, true, EPI_STORE>(dev, dtype, M, N, a, nullptr, b, nullptr, 0, 1,
                                                   ep, 0u, st);
  return launch_gemm<256, true, false, EPI_STORE>(dev, dtype, M, N, a, nullptr, b, nullptr, 0, 1,
                                                  ep, 0u, st);
}

}  // extern "C"

// ------------------------------------- column sums without caller scratch ----
// Scratch for gmlp_colsum_static lives in the library image. The array's name is a
// host-side handle in host code, not a device address: the address kernels can use
// is looked up once per device with cudaGetSymbolAddress (below) and cached.
namespace gmlp {
constexpr size_t COLSUM_STATIC_BYTES = 1u << 20;  // 1 MiB per GPU that loads the library
static __device__ __align__(256) float g_colsum_static_scratch[COLSUM_STATIC_BYTES / sizeof(float)];
static float* g_colsum_static_ptr[64] = {};
static std::mutex g_colsum_static_mu;
}  // namespace gmlp

extern "C" int gmlp_colsum_static(int64_t rows, int64_t cols, int32_t dtype, const void* src,
                                  int64_t ld, void* dst, void* stream) {
  int rc;
  if ((rc = colsum_check(rows, cols, dtype, src, ld, dst))) return rc;
  const size_t need = gmlp_colsum_scratch_bytes(rows, cols);
  if (need > COLSUM_STATIC_BYTES)
    return fail(GMLP_ERR_SCRATCH,
                "rows=%lld cols=%lld needs %zu bytes of partial sums but the built-in scratch of "
                "gmlp_colsum_static holds %zu; use gmlp_colsum with caller-provided scratch",
                static_cast<long long>(rows), static_cast<long long>(cols), need,
                static_cast<size_t>(COLSUM_STATIC_BYTES));
  const DeviceInfo* dev;
  if ((rc = device_info(&dev))) return rc;
  int ordinal = 0;
  cudaError_t e = cudaGetDevice(&ordinal);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  float* part = nullptr;
  {
    // First call on this device: resolve the array's device address, with this
    // device current. Later calls reuse it.
    std::lock_guard<std::mutex> lk(g_colsum_static_mu);
    if (!g_colsum_static_ptr[ordinal]) {
      float* p = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_static_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(GMLP_ERR_LAUNCH, "cudaGetSymbolAddress(colsum scratch): %s",
                    cudaGetErrorString(e));
      g_colsum_static_ptr[ordinal] = p;
    }
    part = g_colsum_static_ptr[ordinal];
  }
  // Nothing left in the array by an earlier call is ever read (see colsum_launch), so
  // nothing has to be cleared.
  return colsum_launch(rows, cols, dtype, src, ld, part, dst, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------- peer memory + all-reduce --
extern "C" size_t gmlp_peer_region_bytes(int64_t max_elems, int32_t world) {
  if (max_elems <= 0 || world < 2 || world > gmlp::PEER_MAX_WORLD) return 0;
  return static_cast<size_t>(gmlp::peer_region_bytes(max_elems, world));
}

extern "C" int gmlp_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  using namespace gmlp;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the ABI carries the handle as 64 opaque bytes");
  if (!ptr || !handle64 || bytes == 0) return fail(GMLP_ERR_ARG, "NULL pointer or zero size");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess)
    return fail(GMLP_ERR_LAUNCH, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(GMLP_ERR_LAUNCH, "peer buffer set-up: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return GMLP_OK;
}

extern "C" int gmlp_peer_open(const void* handle64, void** ptr) {
  using namespace gmlp;
  if (!ptr || !handle64) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess)
    return fail(GMLP_ERR_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *ptr = p;
  return GMLP_OK;
}

extern "C" int gmlp_peer_close(void* ptr) {
  using namespace gmlp;
  if (!ptr) return GMLP_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess)
    return fail(GMLP_ERR_LAUNCH, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

extern "C" int gmlp_peer_free(void* ptr) {
  using namespace gmlp;
  if (!ptr) return GMLP_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "cudaFree: %s", cudaGetErrorString(e));
  return GMLP_OK;
}

// Size from which gmlp_peer_allreduce takes the two-shot form: 0 = built-in rule,
// > 0 = that many bytes at any group size, < 0 = never.
static long long g_two_shot_bytes = 0;
extern "C" long long gmlp_set_peer_two_shot_bytes(long long bytes) {
  const long long prev = g_two_shot_bytes;
  g_two_shot_bytes = bytes;
  return prev;
}

static int peer_allreduce_impl(int32_t dtype, int64_t n, int64_t max_elems, const void* src,
                               void* const* regions, int32_t rank, int32_t world, void* dst,
                               int32_t dependent, bool scattered, void* stream);

extern "C" int gmlp_peer_allreduce(int32_t dtype, int64_t n, int64_t max_elems, const void* src,
                                   void* const* regions, int32_t rank, int32_t world, void* dst,
                                   int32_t dependent, void* stream) {
  return peer_allreduce_impl(dtype, n, max_elems, src, regions, rank, world, dst, dependent, false, stream);
}

extern "C" int gmlp_peer_reduce_gather(int32_t dtype, int64_t n, int64_t max_elems, void* y,
                                       void* const* regions, int32_t rank, int32_t world, void* stream) {
  if (world > 0 && (n % (8ll * world)) != 0)
    return fail(GMLP_ERR_SHAPE, "n=%lld must be a multiple of 8 * world", static_cast<long long>(n));
  return peer_allreduce_impl(dtype, n, max_elems, y, regions, rank, world, y, 0, true, stream);
}

static int peer_allreduce_impl(int32_t dtype, int64_t n, int64_t max_elems, const void* src,
                               void* const* regions, int32_t rank, int32_t world, void* dst,
                               int32_t dependent, bool scattered, void* stream) {
  using namespace gmlp;
  if (dtype != GMLP_BF16 && dtype != GMLP_FP16)
    return fail(GMLP_ERR_DTYPE, "dtype %d is not GMLP_BF16 / GMLP_FP16", dtype);
  if (world < 2 || world > PEER_MAX_WORLD || rank < 0 || rank >= world)
    return fail(GMLP_ERR_ARG, "peer all-reduce needs 2 <= world <= %d and 0 <= rank < world; got rank %d of %d",
                PEER_MAX_WORLD, rank, world);
  if (n <= 0 || (n % 8) != 0 || n > max_elems)
    return fail(GMLP_ERR_SHAPE,
                "peer all-reduce needs a positive element count that is a multiple of 8 and at most the "
                "regions' capacity of %lld; got %lld",
                static_cast<long long>(max_elems), static_cast<long long>(n));
  if (!src || !regions || !dst) return fail(GMLP_ERR_ARG, "NULL pointer argument");
  if (!aligned16(src) || !aligned16(dst))
    return fail(GMLP_ERR_ALIGN, "src and dst must be 16-byte aligned");
  PeerReduceArgs a;
  memset(&a, 0, sizeof(a));
  for (int p = 0; p < world; ++p) {
    if (!regions[p]) return fail(GMLP_ERR_ARG, "NULL region for rank %d", p);
    if (!aligned16(regions[p])) return fail(GMLP_ERR_ALIGN, "region of rank %d must be 16-byte aligned", p);
    a.region[p] = static_cast<char*>(regions[p]);
  }
  const DeviceInfo* dev;
  int rc;
  if ((rc = device_info(&dev))) return rc;
  a.src = src;
  a.dst = dst;
  a.n = n;
  a.max_elems = max_elems;
  a.rank = rank;
  a.world = world;
  a.dependent = dependent ? 1 : 0;
  a.scattered = scattered ? 1 : 0;
  a.status = dev->status_ptr;
  // Kernel and grid depend on n and world alone, so that every rank makes the same
  // choice and block b means the same slice everywhere. The two-shot form (each rank
  // reduces one slice and hands it round) moves world/2 times less data over NVLink but
  // needs a second flag exchange, which pays only for the largest messages on the
  // largest groups: it is taken from PEER_TWO_SHOT_MIN_BYTES on with eight ranks.
  const bool big = g_two_shot_bytes > 0 ? n * 2 >= g_two_shot_bytes
                                        : (g_two_shot_bytes == 0 && world >= 8 && n * 2 >= PEER_TWO_SHOT_MIN_BYTES);
  const bool two_shot = scattered || (big && (n % (8ll * world)) == 0);
  const long long vecs = two_shot ? n / 8 / world : n / 8;
  long long blocks = (vecs + PEER_THREADS - 1) / PEER_THREADS;
  if (blocks > PEER_MAX_BLOCKS) blocks = PEER_MAX_BLOCKS;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(PEER_THREADS);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (dependent) {
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e;
  if (two_shot)
    e = dtype == GMLP_BF16 ? cudaLaunchKernelEx(&cfg, peer_allreduce_twoshot_kernel<__nv_bfloat16>, a)
                           : cudaLaunchKernelEx(&cfg, peer_allreduce_twoshot_kernel<__half>, a);
  else
    e = dtype == GMLP_BF16 ? cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<__nv_bfloat16>, a)
                           : cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<__half>, a);
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GMLP_ERR_LAUNCH, "kernel launch: %s", cudaGetErrorString(e));
  return GMLP_OK;
}
