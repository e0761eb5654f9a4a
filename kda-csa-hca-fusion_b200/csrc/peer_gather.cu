// All-gather of per-GPU head slices by plain peer stores, for the one-token decode step.
//
// Under head sharding every layer ends with an all-gather of `[B, (h/N)*c]` rows before `o_proj`.  At decode sizes
// (B = 64: 256 KiB per layer over all ranks) a library collective is pure latency; here each rank instead writes its
// slab straight into every peer's gather buffer over NVLink (`st.global` to peer-mapped addresses, 16 bytes per
// thread) and the ranks meet on flags that live next to those buffers.  One launch of one CTA per rank:
//   1. arrival: store `seq` into slot `rank` of every peer's arrival flags, then wait until all local slots hold
//      `seq` -- every rank has reached this call, so everything it launched before (the consumers of the previous
//      gather into the same buffer) has finished and the buffer may be overwritten;
//   2. copy the slab into slot `rank` of every peer's buffer (and the own one), `__threadfence_system()`;
//   3. data: store `seq` into slot `rank` of every peer's data flags, wait until all local slots hold `seq`.
// `seq` counts the calls on this buffer and lives in device memory beside the flags, so a replayed CUDA graph needs no
// changing launch argument; all ranks make the same calls, so their counters agree.
// Every wait is bounded: after the limit the kernel records KCH_STATUS_PEER_GATHER in the status word and returns
// (the context stays usable; the gathered data of that call is not valid).  No multicast, no multimem, no library
// kernel touches a peer pointer: plain loads and stores of this kernel only.
//
// Large slabs (the gathers of a prefill pass: tens of megabytes per rank) take the same three steps as three launches on
// the caller's stream: the arrival step (one CTA), a copy kernel of many CTAs that stores the slab to every peer with
// 16-byte stores, and the data-flag step (one CTA); the kernel boundaries order them.
//
// The buffers and flags must be memory that every rank has mapped from every peer (CUDA VMM / IPC; the Python side
// uses torch's symmetric-memory allocator) and zero-initialised flags.  The reference has no counterpart (it has no
// distributed code).
#include <stdint.h>

#include "mma_utils.cuh"

#define PG_MAX_WORLD 16
#define PG_SPIN (1u << 22)

struct PeerGatherArgs {
  const uint4* src;                 // this rank's slab, `slab_bytes` long, 16-byte aligned
  int64_t slab_bytes;
  uint8_t* bufs[PG_MAX_WORLD];      // gather buffer of every rank, as mapped on THIS rank: [world][slab_bytes]
  uint32_t* flags[PG_MAX_WORLD];    // flag block of every rank: [0, world) arrival, [world, 2 world) data, [2 world] seq
  int rank, world;
  int phase;                        // 0: arrival, copy and data flags in this one CTA; 1: arrival only; 2: data flags only
  unsigned int* status;
};

__device__ __forceinline__ void pg_store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t pg_load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// thread p < world waits for slot p of the local flag row; returns false after the poll limit
__device__ __forceinline__ bool pg_wait(const uint32_t* slot, uint32_t seq, unsigned int* status) {
  for (uint32_t it = 0; it < PG_SPIN; ++it) {
    if (pg_load_acquire_sys(slot) == seq) return true;
    if ((it & 1023) == 1023 && *((volatile unsigned int*)status) != 0) return false;
  }
  atomicCAS(status, 0u, (unsigned)KCH_STATUS_PEER_GATHER);
  return false;
}

__global__ void __launch_bounds__(1024) peer_allgather_kernel(PeerGatherArgs a) {
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  uint32_t* mine = a.flags[a.rank];
  const uint32_t seq = mine[2 * a.world] + 1;          // every thread reads the same value; written back at the end
  if (tid == 0) s_ok = 1;
  __syncthreads();
  // 1. arrival
  if (a.phase != 2 && tid < a.world) {
    pg_store_release_sys(a.flags[tid] + a.rank, seq);
    if (!pg_wait(mine + tid, seq, a.status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok || a.phase == 1) return;
  // 2. the slab into slot `rank` of every rank's buffer
  if (a.phase == 0) {
    const int64_t n16 = a.slab_bytes >> 4;
    for (int p = 0; p < a.world; ++p) {
      uint4* dst = reinterpret_cast<uint4*>(a.bufs[p] + (int64_t)a.rank * a.slab_bytes);
      for (int64_t i = tid; i < n16; i += blockDim.x) dst[i] = a.src[i];
    }
    __threadfence_system();
    __syncthreads();
  }
  // 3. data flags
  if (tid < a.world) {
    pg_store_release_sys(a.flags[tid] + a.world + a.rank, seq);
    if (!pg_wait(mine + a.world + tid, seq, a.status)) s_ok = 0;
  }
  __syncthreads();
  if (tid == 0 && s_ok) mine[2 * a.world] = seq;
}

// the copy step of a large gather: grid-stride over 16-byte words, every word stored to each rank's buffer
__global__ void __launch_bounds__(512) peer_allgather_copy_kernel(PeerGatherArgs a) {
  const int64_t n16 = a.slab_bytes >> 4;
  if (*((volatile unsigned int*)a.status) != 0) return;       // the arrival step gave up: leave the peers' buffers alone
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = a.src[i];
    for (int p = 0; p < a.world; ++p)
      reinterpret_cast<uint4*>(a.bufs[p] + (int64_t)a.rank * a.slab_bytes)[i] = v;
  }
}

extern "C" int64_t kch_peer_gather_flag_words(int world) { return world >= 1 ? 2 * (int64_t)world + 2 : 0; }

extern "C" int kch_peer_allgather(const void* src, int64_t slab_bytes, void* const* bufs, void* const* flags, int rank,
                                  int world, void* stream) {
  KCH_REQUIRE(world >= 1 && world <= PG_MAX_WORLD && rank >= 0 && rank < world,
              "kch_peer_allgather: rank=%d world=%d (world <= %d)", rank, world, PG_MAX_WORLD);
  KCH_REQUIRE(src && bufs && flags && slab_bytes >= 16 && (slab_bytes % 16) == 0 && (((uintptr_t)src) & 15) == 0,
              "kch_peer_allgather: the slab must be 16-byte aligned and a multiple of 16 bytes (slab_bytes=%lld)",
              (long long)slab_bytes);
  KCH_REQUIRE(slab_bytes <= (4LL << 30), "kch_peer_allgather: slab_bytes=%lld exceeds 4 GiB", (long long)slab_bytes);
  unsigned int* status = kch_status_device_ptr();
  KCH_REQUIRE(status != nullptr, "kch_peer_allgather: cannot resolve the device status word");
  PeerGatherArgs a = {};
  a.src = (const uint4*)src; a.slab_bytes = slab_bytes; a.rank = rank; a.world = world; a.status = status;
  for (int p = 0; p < world; ++p) {
    KCH_REQUIRE(bufs[p] && flags[p] && (((uintptr_t)bufs[p]) & 15) == 0, "kch_peer_allgather: buffer / flags of rank %d", p);
    a.bufs[p] = (uint8_t*)bufs[p];
    a.flags[p] = (uint32_t*)flags[p];
  }
  if (slab_bytes <= (1LL << 20)) {
    a.phase = 0;
    peer_allgather_kernel<<<1, 1024, 0, kch_stream(stream)>>>(a);
    KCH_LAUNCH_OK();
    return KCH_OK;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    KCH_CUDA_OK(cudaGetDevice(&dev));
    KCH_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  a.phase = 1;
  peer_allgather_kernel<<<1, 1024, 0, kch_stream(stream)>>>(a);
  KCH_LAUNCH_OK();
  peer_allgather_copy_kernel<<<2 * sms, 512, 0, kch_stream(stream)>>>(a);
  KCH_LAUNCH_OK();
  a.phase = 2;
  peer_allgather_kernel<<<1, 1024, 0, kch_stream(stream)>>>(a);
  KCH_LAUNCH_OK();
  return KCH_OK;
}
