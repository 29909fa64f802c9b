// Sum of a small tensor over the GPUs of one NVLink / NVSwitch domain, for the
// tensor-parallel partial outputs of the down projection (a few KB to about 1 MB,
// where a ring's latency dominates). Ranks push data into inbox slots in each
// other's memory (plain peer stores over NVLink, no multicast), raise flags there,
// wait for the peers' flags in their own memory and add in rank order in fp32, so all
// ranks end with identical bits.
//
// Each rank owns one peer-mapped region:
//   inbox   [2 parities][world senders][slot_bytes]   data pushed by the peers
//   flags   [2 phases][world senders][PEER_MAX_BLOCKS] u32   last epoch each sender's block announced
//   epoch   u32   calls completed by this rank;   ticket  u32   blocks of the current call that are done
// The epoch is kept on the device (the last block of a launch to finish publishes
// it), so a launch carries no per-call host state and can be replayed. All ranks
// make the same sequence of calls, hence agree on the epoch e of a call.
//
// One-shot kernel (small n), block b of rank r:
//   1. copies its slice of src into inbox[e & 1][r] of every peer;
//   2. after a block barrier, stores e to flags[0][r][b] of every peer (st.release.sys);
//   3. waits until flags[0][p][b] in its own region has reached e for every peer p
//      (ld.acquire.sys; monotonic compare, so a peer already one call ahead is fine);
//   4. adds src and the world-1 inbox slices and writes dst (dst may alias src).
// Two-shot kernel (larger n, world times less NVLink traffic): the tensor is cut into
// `world` equal slices; rank r pushes slice p of its partial to peer p (steps 1-3),
// reduces its own slice r, writes it to dst and pushes it into every peer's
// inbox[e & 1][r] at slice r's offset, announces on flags[1], waits for the peers'
// flags[1] and copies their reduced slices from its inbox to dst.
//
// Inbox parity e & 1 is written again at call e + 2, which a peer can start only after
// this rank has announced e + 1, i.e. after its launch for e has finished reading:
// two parities suffice and no closing handshake is needed.
//
// Every rank must launch the same kernel with the same grid (functions of n and world
// only). Waits are bounded: on expiry the block records GMLP_DEV_TIMEOUT_PEER and
// returns without writing dst.
#pragma once
#include "decode_stream.cuh"

namespace gmlp {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_MAX_BLOCKS = 128;
constexpr int PEER_THREADS = 512;
constexpr int PEER_SLOT_ALIGN = 256;
constexpr int GMLP_DEV_TIMEOUT_PEER = 4;
constexpr long long PEER_TWO_SHOT_MIN_BYTES = 1024 * 1024;
// About one second at the boost clock: the peers' kernels are launched by their own
// hosts, so the skew between ranks is host scheduling noise, not device time.
constexpr long long PEER_WAIT_LIMIT_CYCLES = 2000000000LL;

__host__ __device__ constexpr long long peer_slot_bytes(long long max_elems) {
  return (max_elems * 2 + PEER_SLOT_ALIGN - 1) / PEER_SLOT_ALIGN * PEER_SLOT_ALIGN;
}
__host__ __device__ constexpr long long peer_flags_offset(long long max_elems, int world) {
  return 2ll * world * peer_slot_bytes(max_elems);
}
__host__ __device__ constexpr long long peer_epoch_offset(long long max_elems, int world) {
  return peer_flags_offset(max_elems, world) + 2ll * 4 * world * PEER_MAX_BLOCKS;
}
__host__ __device__ constexpr long long peer_region_bytes(long long max_elems, int world) {
  return peer_epoch_offset(max_elems, world) + PEER_SLOT_ALIGN;
}

struct PeerReduceArgs {
  char* region[PEER_MAX_WORLD];  // region[p]: rank p's region (peer-mapped for p != rank)
  const void* src;               // this rank's partial
  void* dst;                     // this rank's output (may alias src)
  long long n;                   // elements, a multiple of 8 (of 8 * world for the two-shot kernel)
  long long max_elems;           // the capacity the regions were sized for
  int rank, world;
  int dependent;  // launched as a programmatic dependent of the kernel that wrote src
  int scattered;  // two-shot kernel only: the slices are in the owners' inboxes already (the down
                  // projection pushed them from its epilogue), so the kernel starts at the first flag exchange
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
__device__ __forceinline__ void accumulate8(float (&acc)[8], const uint4& q) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = Pack2<T>::unpack(w[k]);
    acc[2 * k] += f.x;
    acc[2 * k + 1] += f.y;
  }
}

// Start of a call: the epoch of this call, the same in every block (the previous
// launch published its epoch before it ended, and this one starts after it).
__device__ __forceinline__ unsigned int peer_begin(const PeerReduceArgs& a, unsigned int* s_epoch, int* s_abort) {
  // A programmatic dependent that follows (the next weight-streaming kernel) may start
  // prefetching its weights now; its own griddepcontrol.wait still holds it back from
  // anything this kernel writes until this grid has finished.
  if (threadIdx.x == 0) pdl_launch_dependents();
  if (a.dependent) pdl_wait();  // the preceding grid's partial must be complete and visible
  if (threadIdx.x == 0) {
    *s_abort = 0;
    const unsigned int* done = reinterpret_cast<const unsigned int*>(
        a.region[a.rank] + peer_epoch_offset(a.max_elems, a.world));
    *s_epoch = __ldcg(done) + 1u;
  }
  __syncthreads();
  return *s_epoch;
}

// End of a call: the last block to get here publishes the epoch and clears the ticket.
__device__ __forceinline__ void peer_end(const PeerReduceArgs& a, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* done =
        reinterpret_cast<unsigned int*>(a.region[a.rank] + peer_epoch_offset(a.max_elems, a.world));
    unsigned int* ticket = done + 1;
    __threadfence();
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      *done = epoch;
    }
  }
}

// Announce `epoch` on flag array `phase` of every peer, then wait for every peer's
// announcement in this rank's own flags. Called by all threads; returns false when
// the wait ran out.
__device__ __forceinline__ bool peer_exchange(const PeerReduceArgs& a, unsigned int epoch, int phase,
                                              int* s_abort) {
  __syncthreads();  // this block's pushes are issued; the release below publishes them
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const int p = threadIdx.x;
    const long long fo =
        peer_flags_offset(a.max_elems, a.world) + 4ll * phase * a.world * PEER_MAX_BLOCKS;
    st_release_sys(reinterpret_cast<unsigned int*>(a.region[p] + fo) + a.rank * PEER_MAX_BLOCKS + blockIdx.x,
                   epoch);
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(a.region[a.rank] + fo) +
                               p * PEER_MAX_BLOCKS + blockIdx.x;
    const long long t0 = clock64();
    while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
      if (clock64() - t0 > PEER_WAIT_LIMIT_CYCLES) {
        atomicCAS(a.status, 0, GMLP_DEV_TIMEOUT_PEER);
        *s_abort = 1;
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  return *s_abort == 0;
}

template <typename T>
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(PeerReduceArgs a) {
  __shared__ int s_abort;
  __shared__ unsigned int s_epoch;
  const unsigned int epoch = peer_begin(a, &s_epoch, &s_abort);
  char* const mine = a.region[a.rank];
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
  // 2 + 3. flags
  if (peer_exchange(a, epoch, 0, &s_abort)) {
    // 4. rank-ordered fp32 sum of the own partial and the inbox slices
    for (long long v = v0; v < vecs; v += vstep) {
      uint4 q[PEER_MAX_WORLD];
#pragma unroll
      for (int p = 0; p < PEER_MAX_WORLD; ++p) {
        if (p < a.world)
          q[p] = p == a.rank
                     ? src[v]
                     : ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(mine + parity_off + p * slot) + v);
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < PEER_MAX_WORLD; ++p)
        if (p < a.world) accumulate8<T>(acc, q[p]);
      store8(static_cast<T*>(a.dst) + v * 8, acc);
    }
  }
  peer_end(a, epoch);
}

template <typename T>
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_twoshot_kernel(PeerReduceArgs a) {
  __shared__ int s_abort;
  __shared__ unsigned int s_epoch;
  const unsigned int epoch = peer_begin(a, &s_epoch, &s_abort);
  char* const mine = a.region[a.rank];
  const long long slot = peer_slot_bytes(a.max_elems);
  const long long parity_off = static_cast<long long>(epoch & 1u) * a.world * slot;
  const long long svecs = (a.n >> 3) / a.world;  // 16-byte vectors per slice
  const long long v0 = static_cast<long long>(blockIdx.x) * PEER_THREADS + threadIdx.x;
  const long long vstep = static_cast<long long>(gridDim.x) * PEER_THREADS;
  const uint4* src = static_cast<const uint4*>(a.src);
  uint4* dst = static_cast<uint4*>(a.dst);

  // scatter: slice p of this rank's partial goes to peer p (same offset in the slot)
  for (long long v = v0; v < svecs && !a.scattered; v += vstep) {
#pragma unroll
    for (int p = 0; p < PEER_MAX_WORLD; ++p)
      if (p < a.world && p != a.rank)
        reinterpret_cast<uint4*>(a.region[p] + parity_off + a.rank * slot)[p * svecs + v] = src[p * svecs + v];
  }
  if (peer_exchange(a, epoch, 0, &s_abort)) {
    // reduce this rank's slice in rank order; keep it and push it to every peer
    const long long base = a.rank * svecs;
    for (long long v = v0; v < svecs; v += vstep) {
      uint4 q[PEER_MAX_WORLD];
#pragma unroll
      for (int p = 0; p < PEER_MAX_WORLD; ++p) {
        if (p < a.world)
          q[p] = p == a.rank ? src[base + v]
                             : ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(mine + parity_off + p * slot) +
                                                 base + v);
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < PEER_MAX_WORLD; ++p)
        if (p < a.world) accumulate8<T>(acc, q[p]);
      uint4 r;
      r.x = Pack2<T>::pack(acc[0], acc[1]);
      r.y = Pack2<T>::pack(acc[2], acc[3]);
      r.z = Pack2<T>::pack(acc[4], acc[5]);
      r.w = Pack2<T>::pack(acc[6], acc[7]);
      dst[base + v] = r;
#pragma unroll
      for (int p = 0; p < PEER_MAX_WORLD; ++p)
        if (p < a.world && p != a.rank)
          reinterpret_cast<uint4*>(a.region[p] + parity_off + a.rank * slot)[base + v] = r;
    }
    if (peer_exchange(a, epoch, 1, &s_abort)) {
      // gather: the peers' reduced slices have arrived in this rank's inbox
      for (long long v = v0; v < svecs; v += vstep) {
#pragma unroll
        for (int p = 0; p < PEER_MAX_WORLD; ++p)
          if (p < a.world && p != a.rank)
            dst[p * svecs + v] =
                ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(mine + parity_off + p * slot) + p * svecs + v);
      }
    }
  }
  peer_end(a, epoch);
}

}  // namespace gmlp
