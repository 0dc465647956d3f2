// sm_100a building blocks used by every kernel in this library: mbarrier with bounded waits,
// TMA tile loads (never multicast), tcgen05 MMA / TMEM load-store, and the shared-memory matrix
// and instruction descriptors that tcgen05.mma consumes.  Hand-written inline PTX; no CUTLASS.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace da {

// ---------------------------------------------------------------------------------------------
// Device-side status word.  A wait that gives up records where it was and the kernel unwinds
// through its normal teardown (TMEM is freed, no trap).  The host reads it with diffattn_status().
// ---------------------------------------------------------------------------------------------
__device__ int g_status[4];   // [0] = first failing wait site (0 = OK), [1] = blockIdx.x, [2] = blockIdx.y, [3] = iteration

static constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s per wait, then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 r;\n\t"
      "elect.sync r|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// Register re-allocation between the roles of a warp-specialised CTA.  Every warp of a warpgroup (four consecutive
// warps) must execute the same instruction.  Registers only move inside the pool the CTA was launched with, which
// is kept per scheduler: for every scheduler, the sum over its warps of the new per-thread counts must not exceed
// (warps on that scheduler) x (registers per thread at launch); an increase that cannot be satisfied blocks for ever.
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ------------------------------------------ mbarrier -----------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// (One arrival per warp -- __syncwarp, then lane 0 arrives -- instead of one per thread was measured in every
// kernel of the default path: forward +0.7 %, dK/dV -1 %, dQ +6 % at B4 H16 N4096 D64.  The converging step delays the
// arrival of the warp's fastest threads; per-thread arrivals stay.)
// Suspend-time hint: the hardware may park the waiting thread for up to this long (it is woken when the
// phase completes) instead of returning at once to be polled again.
static constexpr uint32_t kSuspendHintNs = 1000000u;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

// Non-blocking look at a phase.  A wait on an mbarrier costs the waiting thread 100-350 clocks even when the phase
// completed long ago (more, the busier shared memory is).  Where the phase is very likely complete, a role probes it
// a stretch of independent work BEFORE it needs the answer and falls back to mbar_wait only if the probe said no: the
// probe's latency then overlaps that work.  (A true answer stays true until the waiter itself lets the next phase
// start.)
__device__ __forceinline__ uint32_t mbar_probe(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  `abort_flag` lives in shared memory; once any role gives up, every other wait in
// the CTA returns false at its next poll so that the whole CTA reaches its teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int site,
                                          int iter = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (atomicCAS(&g_status[0], 0, site) == 0) {
          g_status[1] = blockIdx.x;
          g_status[2] = blockIdx.y;
          g_status[3] = iter;
        }
        return false;
      }
    }
  }
}

// (Polling with mbarrier.test_wait instead of the parking try_wait was measured on the forward's hand-overs:
// no gain, the polling warps take issue slots from the working ones.)

// Same wait executed by a whole converged warp; the result is made warp-uniform so that the warp
// stays converged (elect.sync below needs all 32 lanes) even when a wait gives up.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int site,
                                               int iter = 0) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, site, iter));
}

// ---------------------------------- thread-block clusters ----------------------------------
// The partner CTA's shared memory (distributed shared memory): a local shared-memory address mapped into CTA `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_st_v4(uint32_t remote_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// arrival on an mbarrier of the partner CTA; releases this thread's earlier writes (to either CTA) at cluster scope
__device__ __forceinline__ void cluster_mbar_arrive(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr) : "memory");
}
// whole cluster: every thread of both CTAs arrives, then waits (like __syncthreads over the cluster)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bounded wait on a LOCAL mbarrier whose arrivals come from the partner CTA: acquire at cluster scope, so that the
// partner's distributed-shared-memory writes before its arrival are visible afterwards.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int site, int iter = 0) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    if (ok) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (atomicCAS(&g_status[0], 0, site) == 0) {
          g_status[1] = blockIdx.x;
          g_status[2] = blockIdx.y;
          g_status[3] = iter;
        }
        return false;
      }
    }
  }
}

// named barrier among `nthreads` threads of the CTA (id 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// non-blocking arrival on a named barrier: lets a warp that has given up (a bounded wait expired) stand in for the
// bar.sync calls it will no longer make, so that a partner still running its loop is never left waiting on it
__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// --------------------------------------------- TMA -------------------------------------------
// 4-D tiled load global -> shared, completion counted in bytes on an mbarrier.  No multicast.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 4-D tiled store shared -> global (bulk-group completion).  The engine clips the box at the tensor's bounds, so
// rows past the sequence end and columns past a narrow head are simply not written.  Coordinates must be >= 0.
__device__ __forceinline__ void tma_store_4d(const void* smem_src, const CUtensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// returns once the engine has read the shared-memory sources of every committed store (the global writes
// themselves complete by the end of the kernel)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// One 16-byte chunk of a [rows][64 x 16-bit] tile in the 128-byte-swizzled layout TMA and the MMA descriptors
// use: row r occupies 128 bytes, chunk c of it sits at position c ^ (r & 7).  The tile base is 1024-aligned.
__device__ __forceinline__ void st_swizzled_chunk(uint8_t* tile, int r, int c, uint4 v) {
  *reinterpret_cast<uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// untiled bulk copy global -> shared (addresses 16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ------------------------------------------- tcgen05 -----------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {       // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]      (one thread issues)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
// mbarrier arrives once every tcgen05 op issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Instruction descriptor, kind::f16, A and B both fp16 or both bf16, fp32 accumulate.
//   [4,6) D format (1 = f32)  [7,10) A format (0 = f16, 1 = bf16)  [10,13) B format (same)
//   [15] A major (0 = K, 1 = MN)  [16] B major  [17,23) N>>3  [24,29) M>>4
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_mn_major, int b_mn_major, bool bf16 = false) {
  return (1u << 4) | (uint32_t(bf16) << 7) | (uint32_t(bf16) << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.
//   [0,14) start>>4  [16,30) leading byte offset>>4  [32,46) stride byte offset>>4
//   [46,48) version = 1  [61,64) layout (2 = SWIZZLE_128B)
// K-major operand (rows of 64 halves = 128 B, 8-row swizzle atoms 1024 B apart): SBO = 1024, LBO unused.
// MN-major operand (atoms of 64 MN elements x 8 K rows): LBO = byte distance between atoms along MN,
// SBO = byte distance between 8-row groups along K.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3ffff) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}
__device__ __forceinline__ uint64_t sdesc_kmajor(uint32_t smem_addr) { return make_sdesc(smem_addr, 16, 1024); }

// Lean forms for issuer loops.  Every descriptor used by this library has SBO = 1024, version 1 and
// SWIZZLE_128B, so the upper 32 bits are one constant and only the lower word (start address and LBO)
// changes: advancing an operand is a 32-bit add of (bytes >> 4).
static constexpr uint32_t kSdescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t sdesc_lo(uint32_t smem_addr, uint32_t lbo_bytes = 16) {
  return ((smem_addr & 0x3ffffu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accum), "r"(kSdescHi)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accum), "r"(kSdescHi)
      : "memory");
}

// ---- TMEM <-> registers, shape 32x32b: thread t of warp w touches lane 32*(w%4)+t, one column per register
#define DA_R4(r, i) "=r"(r[i]), "=r"(r[i + 1]), "=r"(r[i + 2]), "=r"(r[i + 3])
#define DA_W4(r, i) "r"(r[i]), "r"(r[i + 1]), "r"(r[i + 2]), "r"(r[i + 3])

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : DA_R4(r, 0), DA_R4(r, 4), DA_R4(r, 8), DA_R4(r, 12)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : DA_R4(r, 0), DA_R4(r, 4), DA_R4(r, 8), DA_R4(r, 12), DA_R4(r, 16), DA_R4(r, 20), DA_R4(r, 24), DA_R4(r, 28)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), DA_W4(r, 0), DA_W4(r, 4), DA_W4(r, 8), DA_W4(r, 12)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), DA_W4(r, 0), DA_W4(r, 4), DA_W4(r, 8), DA_W4(r, 12), DA_W4(r, 16), DA_W4(r, 20), DA_W4(r, 24),
      DA_W4(r, 28)
      : "memory");
}

// Packed fp32 pairs (one 64-bit register, two lanes): sm_100 issues an fma/mul/add on both halves as ONE instruction,
// which halves the issue slots of the elementwise passes that surround the exponentials.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f32x2 pk2u(uint32_t lo, uint32_t hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void up2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// (2^x on the FMA and integer pipes -- round-to-nearest split by the 1.5*2^23 trick, degree-3 minimax of 2^f on
// [-0.5, 0.5] with relative error 7.5e-5, exponent added as an integer -- was measured in place of every 2nd, 3rd,
// 4th and 8th exponential of the forward: 1.17, 1.08, 1.04, 0.99 ms against 0.975 ms with the exp unit alone.  The
// kernels are bound by instruction issue around the exp unit, not by the unit's rate.  With the packed f32x2
// instructions the routine costs 10 instructions per pair; every 3rd, 4th, 6th pair of the forward then measured
// 0.825, 0.821, 0.804 ms against 0.804 ms without it.  The routine is not kept.)
// the same, pinned in program order relative to other volatile statements (barrier arrivals between two groups of them)
__device__ __forceinline__ float ex2v(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 16-bit storage type of the tensors: BF = false fp16, BF = true bf16.  Two floats -> one packed word
// (lo in the low half), round to nearest even, and back; one raw 16-bit element <-> float.
template <bool BF>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    return pack_half2(lo, hi);
  }
}
template <bool BF>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF>
__device__ __forceinline__ float to_float16b(__half raw) {      // raw: 16 bits of either type
  if constexpr (BF) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw));
  else return __half2float(raw);
}
template <bool BF>
__device__ __forceinline__ __half from_float16b(float x) {
  if constexpr (BF) { __nv_bfloat16 b = __float2bfloat16_rn(x); return *reinterpret_cast<__half*>(&b); }
  else return __float2half_rn(x);
}

// ------------------------------------------ attention dropout ------------------------------------------
// Counter-based keep mask: nothing is stored, every kernel recomputes the decisions it needs.  One 32-bit hash
// serves a 2 x 2 block of (query row, key column) positions, one byte per position, so that a thread walking
// along a row (forward, dQ) and a thread walking down a column (dK/dV) both get two decisions per hash:
//   h    = mix32( ((row >> 1) << 16 | (col >> 1)) ^ key ),  key = drop_key(seed, batch*head index, branch)
//   keep = byte (row & 1) * 2 + (col & 1) of h  >=  threshold        (threshold = round(256 p), 1..255)
// mix32 is the two-multiply xorshift finaliser "lowbias32" (C. Wellons, public domain).  Kept probabilities
// are multiplied by 256 / (256 - threshold).  The CPU oracle restates exactly this.
__host__ __device__ __forceinline__ uint32_t mix32(uint32_t h) {
  h ^= h >> 16; h *= 0x7feb352dU; h ^= h >> 15; h *= 0x846ca68bU; h ^= h >> 16;
  return h;
}
__host__ __device__ __forceinline__ uint32_t drop_key(uint32_t seed_lo, uint32_t seed_hi, uint32_t bh, uint32_t branch) {
  return mix32(seed_lo ^ mix32(seed_hi + 0x9E3779B9U * (2u * bh + branch + 1u)));
}
__device__ __forceinline__ uint32_t drop_hash(uint32_t key, uint32_t row2, uint32_t col2) {
  return mix32(((row2 << 16) | col2) ^ key);
}
__device__ __forceinline__ bool drop_keep(uint32_t h, int byte, uint32_t thresh) { return ((h >> (8 * byte)) & 0xffu) >= thresh; }
// mask for one packed pair of 16-bit probabilities of ONE row (columns 2c, 2c+1): bytes 2*(row&1), 2*(row&1)+1
__device__ __forceinline__ uint32_t drop_pair_mask(uint32_t h, int row_odd, uint32_t thresh) {
  const uint32_t f = row_odd ? (h >> 16) : (h & 0xffffu);
  return ((f & 0xffu) >= thresh ? 0x0000ffffu : 0u) | (f >= (thresh << 8) ? 0xffff0000u : 0u);
}

}  // namespace da
