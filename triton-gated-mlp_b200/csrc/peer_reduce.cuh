// One-shot sum of a small tensor over the GPUs of one NVLink / NVSwitch domain,
// for the tensor-parallel partial outputs of the down projection (a few KB to
// about 1 MB, where a ring's latency dominates). Every rank pushes its partial into
// an inbox slot in each peer's memory (plain peer stores over NVLink, no multicast),
// raises a flag there, waits for the peers' flags in its own memory and adds the
// world partials in rank order in fp32, so all ranks end with identical bits.
//
// Each rank owns one peer-mapped region:
//   inbox    [2 parities][world senders][slot_bytes]   partials pushed by the peers
//   flags    [world senders][PEER_MAX_BLOCKS] u32       last epoch each sender's block announced
//   counters [PEER_MAX_BLOCKS] u32                      this rank's own epoch per block
// The epoch is kept on the device (block b bumps counters[b] once per launch), so a
// launch carries no per-call host state and the same launch can be replayed. All
// ranks make the same sequence of calls, hence agree on the epoch.
//
// Per launch, block b of rank r, epoch e:
//   1. copies its slice of src into inbox[e & 1][r] of every peer;
//   2. after a block barrier, stores e to flags[r][b] of every peer (st.release.sys);
//   3. waits until flags[p][b] in its own region has reached e for every peer p
//      (ld.acquire.sys; monotonic compare, so a peer already one call ahead is fine);
//   4. adds src and the world-1 inbox slices and writes dst (dst may alias src).
// Inbox parity e & 1 is written again at epoch e + 2, which a peer can reach only
// after this rank has announced e + 1, i.e. after its launch for e has finished
// reading: two parities suffice and no closing handshake is needed.
//
// Every rank must launch the same grid (a function of n only). The wait is bounded:
// on expiry the block records GMLP_DEV_TIMEOUT_PEER and returns without writing dst.
#pragma once
#include "decode_stream.cuh"

namespace gmlp {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_MAX_BLOCKS = 64;
constexpr int PEER_THREADS = 512;
constexpr int PEER_SLOT_ALIGN = 256;
constexpr int GMLP_DEV_TIMEOUT_PEER = 4;
// About one second at the boost clock: the peers' kernels are launched by their own
// hosts, so the skew between ranks is host scheduling noise, not device time.
constexpr long long PEER_WAIT_LIMIT_CYCLES = 2000000000LL;

__host__ __device__ constexpr long long peer_slot_bytes(long long max_elems) {
  return (max_elems * 2 + PEER_SLOT_ALIGN - 1) / PEER_SLOT_ALIGN * PEER_SLOT_ALIGN;
}
__host__ __device__ constexpr long long peer_flags_offset(long long max_elems, int world) {
  return 2ll * world * peer_slot_bytes(max_elems);
}
__host__ __device__ constexpr long long peer_counters_offset(long long max_elems, int world) {
  return peer_flags_offset(max_elems, world) + 4ll * world * PEER_MAX_BLOCKS;
}
__host__ __device__ constexpr long long peer_region_bytes(long long max_elems, int world) {
  return peer_counters_offset(max_elems, world) + 4ll * PEER_MAX_BLOCKS;
}

struct PeerReduceArgs {
  char* region[PEER_MAX_WORLD];  // region[p]: rank p's region (peer-mapped for p != rank)
  const void* src;               // this rank's partial
  void* dst;                     // this rank's output (may alias src)
  long long n;                   // elements, a multiple of 8
  long long max_elems;           // the capacity the regions were sized for
  int rank, world;
  int dependent;  // launched as a programmatic dependent of the kernel that wrote src
  int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 16 bytes of an inbox slot; system scope so that the line is never served from an
// L1 copy left by an earlier epoch of the same parity.
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(PeerReduceArgs a) {
  __shared__ int s_abort;
  __shared__ unsigned int s_epoch;
  char* const mine = a.region[a.rank];
  // A programmatic dependent that follows (the next weight-streaming kernel) may start
  // prefetching its weights now; its own griddepcontrol.wait still holds it back from
  // anything this kernel writes until this grid has finished.
  if (threadIdx.x == 0) pdl_launch_dependents();
  if (a.dependent) pdl_wait();  // the preceding grid's partial must be complete and visible
  if (threadIdx.x == 0) {
    s_abort = 0;
    unsigned int* counter =
        reinterpret_cast<unsigned int*>(mine + peer_counters_offset(a.max_elems, a.world)) + blockIdx.x;
    const unsigned int e = *counter + 1u;
    *counter = e;
    s_epoch = e;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  const long long slot = peer_slot_bytes(a.max_elems);
  const long long parity_off = static_cast<long long>(epoch & 1u) * a.world * slot;
  const long long vecs = a.n >> 3;
  const long long v0 = static_cast<long long>(blockIdx.x) * PEER_THREADS + threadIdx.x;
  const long long vstep = static_cast<long long>(gridDim.x) * PEER_THREADS;
  const uint4* src = static_cast<const uint4*>(a.src);

  // 1. push this block's slice into every peer's inbox
  for (long long v = v0; v < vecs; v += vstep) {
    const uint4 q = src[v];
#pragma unroll
    for (int p = 0; p < PEER_MAX_WORLD; ++p)
      if (p < a.world && p != a.rank)
        reinterpret_cast<uint4*>(a.region[p] + parity_off + a.rank * slot)[v] = q;
  }
  __syncthreads();
  // 2 + 3. announce to peer p, then wait for peer p's announcement
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const int p = threadIdx.x;
    const long long fo = peer_flags_offset(a.max_elems, a.world);
    st_release_sys(reinterpret_cast<unsigned int*>(a.region[p] + fo) + a.rank * PEER_MAX_BLOCKS + blockIdx.x,
                   epoch);
    const unsigned int* flag =
        reinterpret_cast<const unsigned int*>(mine + fo) + p * PEER_MAX_BLOCKS + blockIdx.x;
    const long long t0 = clock64();
    while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
      if (clock64() - t0 > PEER_WAIT_LIMIT_CYCLES) {
        atomicCAS(a.status, 0, GMLP_DEV_TIMEOUT_PEER);
        s_abort = 1;
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  if (s_abort != 0) return;

  // 4. rank-ordered fp32 sum of the own partial and the inbox slices
  for (long long v = v0; v < vecs; v += vstep) {
    uint4 q[PEER_MAX_WORLD];
#pragma unroll
    for (int p = 0; p < PEER_MAX_WORLD; ++p) {
      if (p < a.world)
        q[p] = p == a.rank ? src[v] : ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(mine + parity_off + p * slot) + v);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int p = 0; p < PEER_MAX_WORLD; ++p) {
      if (p < a.world) {
        const uint32_t w[4] = {q[p].x, q[p].y, q[p].z, q[p].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = Pack2<T>::unpack(w[k]);
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      }
    }
    store8(static_cast<T*>(a.dst) + v * 8, acc);
  }
}

}  // namespace gmlp
