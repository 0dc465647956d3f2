// Differential-attention backward for sm_100a, head dims 32 and 64: ONE pass over the score tiles that produces
// dK1, dK2, dV and dQ1, dQ2 (the reference's single loop, src/kernel.py:410-436, without its second computation
// of S and dP at :426-436).
//
// One CTA = 128 key/value rows of one (batch, head); query tiles of 64 rows stream by.  Per tile:
//   S1^T = K1 Q1^T, S2^T = K2 Q2^T, dP^T = V dA^T          (tensor cores, fp32 in TMEM)
//   P_b^T = 2^(s S_b^T - lse_b), Pc = P1 - lam P2, dS_b^T = +-P_b (dP - E_b)    (CUDA cores, thread = key row)
//   dV  += Pc dA,  dK_b += dS_b^T Q_b    (Pc, dS_b^T as K-major A operands from shared-memory tiles [key][query])
//   dQ_b(tile) = dS_b K_b                (the same dS_b^T tiles read as MN-major A operands of M = 64 MMAs)
// The dQ tile of a key block is a partial sum: four drain warps read it from TMEM and add it with
// red.global.add.v4.f32 into an fp32 [2][B*H][N_pad][64] workspace (zeroed by the preprocess kernel); a small
// kernel scales and converts it afterwards.  The sum over key blocks therefore depends on the order in which
// the CTAs of a head arrive (race-free, but not bit-reproducible); dK1, dK2, dV have one owner and a fixed order.
//
// This form is an option (DiffAttnParams.single_pass), not the default: at B4 H16 N4096 D64 it runs in 2.55 ms
// against 2.00 ms for the two-kernel form (bwd.cuh).  What bounds both is shared-memory bandwidth (128 B/clock/SM):
// with 64-column tiles every MMA re-reads its operands, 240 KB per (128 key x 64 query) tile here (S^T 48, dP^T 48,
// dV 32, dK 48, dQ 64) plus 48 KB of operand stores and 33 KB of TMA writes -- as many bytes as the two kernels of
// the other form move together, so removing the second computation of S and dP (8 of 28 MMA units, 2 of 6 N^2
// exponentials) buys no time, and the adds come on top: without them the kernel takes 1.74 ms, with the address
// pattern an ideal drain would have (8 lanes on 128 contiguous bytes; here every lane owns a row) 2.01 ms.
//
// TMEM (512 columns): dV [0,128) dK1 [128,192) dK2 [192,256) | S1^T [256,320) S2^T [320,384) dP^T [384,448):
// the warpgroups pull a tile's scores into registers and release the columns at once, so the score MMAs of tile
// i+1 run under the elementwise work of tile i | dQ tile [448,512): an M = 64 accumulator occupies lanes 0-15 of
// each 32-lane quarter (row r -> lane 32 (r / 16) + r % 16); dQ1 sits there and dQ2 in lanes 16-31 of the same columns.
#pragma once
#include "bwd.cuh"

namespace da {
namespace fused64 {
constexpr int BKV = 128, BQ = 64, HD = 64, DV = 128, ST = 3;
constexpr int K_BYTES = BKV * HD * 2;       // 16 KB
constexpr int V_BYTES = BKV * DV * 2;       // 32 KB, two boxes of 16 KB
constexpr int Q_BYTES = BQ * HD * 2;        // 8 KB
constexpr int DA_BYTES = BQ * DV * 2;       // 16 KB, two boxes of 8 KB
constexpr int STAT_BYTES = BQ * 16;         // 1 KB
constexpr int STAGE_BYTES = 2 * Q_BYTES + DA_BYTES + STAT_BYTES;   // 33 KB
constexpr int PC_BYTES = BKV * BQ * 2;      // 16 KB: [128 key rows][64 query columns], 128-byte swizzled rows
constexpr int OFF_K1 = 0, OFF_K2 = K_BYTES, OFF_V = 2 * K_BYTES;
constexpr int OFF_PC = OFF_V + V_BYTES;                            // 64 KB
constexpr int OFF_DS1 = OFF_PC + PC_BYTES, OFF_DS2 = OFF_DS1 + PC_BYTES;
constexpr int OFF_STAGE = OFF_DS2 + PC_BYTES;                      // 112 KB
constexpr int OFF_MISC = OFF_STAGE + ST * STAGE_BYTES;             // 211 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int NWG = 4;                      // elementwise warpgroups; warpgroup g owns query columns [16g, 16g+16)
// warps 0-15 elementwise; 16 TMA; 17 S^T issuer; 18 dP^T and dQ issuer; 19 dV and dK issuer; 20-23 dQ drain (one per
// TMEM quarter)
constexpr int NUM_THREADS = NWG * 128 + 128 + 128;
constexpr int WARP_TMA = 16, WARP_S = 17, WARP_P = 18, WARP_O = 19, WARP_DRAIN = 20;
constexpr int T_DV = 0, T_DK1 = 128, T_DK2 = 192, T_S1 = 256, T_S2 = 320, T_DP = 384, T_DQ = 448;
// Registers per thread after the role split.  setmaxnreg moves registers inside the pool the CTA was launched with
// (768 threads x 80 registers, the most a 768-thread CTA can get), and an increase that the pool cannot satisfy
// blocks for ever: the three shares must fit.
#ifndef DA_REGS_ELEM
#define DA_REGS_ELEM 96
#define DA_REGS_ROLE 56
#define DA_REGS_DRAIN 40
#endif
constexpr int REGS_LAUNCH = 80;
constexpr int REGS_ELEM = DA_REGS_ELEM, REGS_ROLE = DA_REGS_ROLE, REGS_DRAIN = DA_REGS_DRAIN;
static_assert(NWG * 128 * REGS_ELEM + 128 * REGS_ROLE + 128 * REGS_DRAIN <= NUM_THREADS * REGS_LAUNCH,
              "setmaxnreg shares exceed the CTA's register pool");
static_assert(REGS_ELEM >= REGS_LAUNCH && REGS_ROLE <= REGS_LAUNCH && REGS_DRAIN <= REGS_LAUNCH, "inc / dec directions");
struct Misc {
  uint64_t bar_kv;
  uint64_t full[ST], empty[ST];
  uint64_t s_full;      // S1^T, S2^T and dP^T of a tile written (two committing issuers)
  uint64_t s_free;      // the scores of a tile are in registers (one arrival per elementwise warp)
  uint64_t e_done;      // Pc, dS1^T, dS2^T of a tile are in shared memory (one arrival per elementwise warp)
  uint64_t o_done;      // dV, dK and dQ MMAs of a tile completed: the three shared-memory tiles are reusable (2 commits)
  uint64_t dq_full;     // dQ tile in TMEM complete
  uint64_t dq_free;     // dQ tile is in the drain warps' registers (4 arrivals)
  uint64_t acc_full;
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace fused64

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <bool BF, bool DROP>
__global__ void __launch_bounds__(fused64::NUM_THREADS, 1)
diffattn_bwd_fused64_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                            const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                            const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_da,
                            const __grid_constant__ CUtensorMap tm_dk1, const __grid_constant__ CUtensorMap tm_dk2,
                            const __grid_constant__ CUtensorMap tm_dv, const BwdArgs args) {
  using namespace fused64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, bh = blockIdx.y;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  // Query tiles: the last ones may reach past N (zero dA, neutral statistics).  Under the causal mask only the
  // tiles from the diagonal on see these keys.  Without it every key block visits all nq tiles, starting at a
  // tile that depends on the key block (tile (i + shift) % nq at step i), so that the key blocks of a head,
  // which start together, add their dQ partial sums to different rows at any one time.
  const int nq_all = args.n_pad / BQ;
  const int i0 = args.causal ? kv_tile * (BKV / BQ) : 0;
  const int nq = nq_all - i0;
  const int shift = !args.causal ? (kv_tile * (BKV / BQ)) % nq : 0;
  auto tile_of = [&](int i) { int t = i + shift; if (t >= nq) t -= nq; return i0 + t; };

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_kv, 1);
    for (int i = 0; i < ST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->empty[i], 1); }
    mbar_init(&misc->s_full, 2);
    mbar_init(&misc->s_free, NWG * 4);
    mbar_init(&misc->e_done, NWG * 4);
    mbar_init(&misc->o_done, 2);
    mbar_init(&misc->dq_full, 1);
    mbar_init(&misc->dq_free, 4);
    mbar_init(&misc->acc_full, 2);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == WARP_S) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp >= WARP_TMA && warp < WARP_DRAIN) {
    reg_dec<REGS_ROLE>();
    if (warp == WARP_TMA) {
      if (elect_one()) {
        mbar_expect_tx(&misc->bar_kv, 2 * K_BYTES + V_BYTES);
        tma_load_4d(smem + OFF_K1, &tm_k1, &misc->bar_kv, 0, kv_tile * BKV, h_idx, b_idx);
        tma_load_4d(smem + OFF_K2, &tm_k2, &misc->bar_kv, 0, kv_tile * BKV, h_idx, b_idx);
        tma_load_4d(smem + OFF_V, &tm_v, &misc->bar_kv, 0, kv_tile * BKV, h_idx, b_idx);
        tma_load_4d(smem + OFF_V + V_BYTES / 2, &tm_v, &misc->bar_kv, 64, kv_tile * BKV, h_idx, b_idx);
        for (int i = 0; i < nq; ++i) {
          const int st = i % ST;
          uint8_t* sp = smem + OFF_STAGE + st * STAGE_BYTES;
          const int q0 = tile_of(i) * BQ;
          if (!mbar_wait(&misc->empty[st], ((i / ST) & 1) ^ 1, abort_flag, 1401, i)) break;
          mbar_expect_tx(&misc->full[st], STAGE_BYTES);
          tma_load_4d(sp, &tm_q1, &misc->full[st], 0, q0, h_idx, b_idx);
          tma_load_4d(sp + Q_BYTES, &tm_q2, &misc->full[st], 0, q0, h_idx, b_idx);
          tma_load_4d(sp + 2 * Q_BYTES, &tm_da, &misc->full[st], 0, q0, bh, 0);
          tma_load_4d(sp + 2 * Q_BYTES + DA_BYTES / 2, &tm_da, &misc->full[st], 64, q0, bh, 0);
          bulk_load_1d(sp + 2 * Q_BYTES + DA_BYTES, args.stats + (size_t(bh) * args.n_pad + size_t(q0)), STAT_BYTES,
                       &misc->full[st]);
        }
      }
    } else if (warp == WARP_S) {
      // ---- S^T issuer: S1^T, S2^T of tile i+1 as soon as the warpgroups hold the scores of tile i in registers
      if (elect_one()) {
        constexpr uint32_t IDESC_S = make_idesc(BKV, BQ, 0, 0, BF);     // S^T = K Q^T
        const uint32_t k1_lo = sdesc_lo(smem_u32(smem + OFF_K1)), k2_lo = sdesc_lo(smem_u32(smem + OFF_K2));
        const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
        const uint32_t tb = tmem_base;
        auto issue = [&](uint32_t sp_lo) {
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) mma_ss_lo(tb + T_S1, k1_lo + k * 2, sp_lo + k * 2, IDESC_S, k > 0);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) mma_ss_lo(tb + T_S2, k2_lo + k * 2, sp_lo + (Q_BYTES >> 4) + k * 2, IDESC_S, k > 0);
          mma_commit(&misc->s_full);      // two arrivals per tile: this warp's and the dP^T issuer's
        };
        bool ok = mbar_wait(&misc->bar_kv, 0, abort_flag, 1501);
        ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 1502);
        if (ok) {
          tc_fence_after();
          issue(st_lo0);
          int st = 0;
          uint32_t st_par = 0;
          for (int i = 0; i + 1 < nq; ++i) {
            if (++st == ST) { st = 0; st_par ^= 1; }
            if (!mbar_wait(&misc->full[st], st_par, abort_flag, 1503, i)) break;
            if (!mbar_wait(&misc->s_free, i & 1, abort_flag, 1504, i)) break;
            tc_fence_after();
            issue(st_lo0 + st * (STAGE_BYTES >> 4));
          }
        }
      }
    } else if (warp == WARP_P) {
      // ---- dP^T and dQ issuer.  In time order: scores of tile i in registers (s_free(i), early in the warpgroups'
      // pass over tile i) -> dP^T(i+1); operands of tile i written (e_done(i), at the end of that pass) -> dQ(i).
      if (elect_one()) {
        constexpr uint32_t IDESC_S = make_idesc(BKV, BQ, 0, 0, BF);     // dP^T = V dA^T
        constexpr uint32_t IDESC_DQ = make_idesc(BQ, HD, 1, 1, BF);     // dQ_b = dS_b K_b    (M = 64; dS_b^T and K_b MN-major)
        const uint32_t v_lo = sdesc_lo(smem_u32(smem + OFF_V));
        const uint32_t ds1_lo = sdesc_lo(smem_u32(smem + OFF_DS1)), ds2_lo = sdesc_lo(smem_u32(smem + OFF_DS2));
        const uint32_t k1_lo = sdesc_lo(smem_u32(smem + OFF_K1)), k2_lo = sdesc_lo(smem_u32(smem + OFF_K2));
        const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
        const uint32_t tb = tmem_base;
        auto issue_dp = [&](uint32_t sp_lo) {
#pragma unroll
          for (int k = 0; k < DV / 16; ++k)
            mma_ss_lo(tb + T_DP, v_lo + (k / 4) * ((V_BYTES / 2) >> 4) + (k % 4) * 2,
                      sp_lo + ((2 * Q_BYTES) >> 4) + (k / 4) * ((DA_BYTES / 2) >> 4) + (k % 4) * 2, IDESC_S, k > 0);
          mma_commit(&misc->s_full);
        };
        bool ok = mbar_wait(&misc->bar_kv, 0, abort_flag, 1511);
        ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 1512);
        if (ok) {
          tc_fence_after();
          issue_dp(st_lo0);
          int st = 0;
          uint32_t st_par = 0;
          for (int i = 0; i < nq; ++i) {
            if (++st == ST) { st = 0; st_par ^= 1; }
            if (i + 1 < nq) {
              if (!mbar_wait(&misc->full[st], st_par, abort_flag, 1513, i)) break;
              if (!mbar_wait(&misc->s_free, i & 1, abort_flag, 1514, i)) break;
              tc_fence_after();
              issue_dp(st_lo0 + st * (STAGE_BYTES >> 4));
            }
            if (!mbar_wait(&misc->e_done, i & 1, abort_flag, 1515, i)) break;
            if (i > 0) {
              if (!mbar_wait(&misc->dq_free, (i - 1) & 1, abort_flag, 1516, i)) break;
            }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              mma_ss_lo(tb + T_DQ, ds1_lo + k * (2048 >> 4), k1_lo + k * (2048 >> 4), IDESC_DQ, k > 0);
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              mma_ss_lo(tb + T_DQ + (16u << 16), ds2_lo + k * (2048 >> 4), k2_lo + k * (2048 >> 4), IDESC_DQ, k > 0);
            mma_commit(&misc->dq_full);
            mma_commit(&misc->o_done);
          }
        }
        mma_commit(&misc->acc_full);
      }
    } else {
      // ---- dV and dK issuer: dV += Pc dA, dK_b += dS_b^T Q_b once the warpgroups have written the operand tiles
      if (elect_one()) {
        constexpr uint32_t IDESC_DV = make_idesc(BKV, DV, 0, 1, BF);    // Pc K-major, dA MN-major
        constexpr uint32_t IDESC_DK = make_idesc(BKV, HD, 0, 1, BF);    // dS^T K-major, Q MN-major
        const uint32_t pc_lo = sdesc_lo(smem_u32(smem + OFF_PC));
        const uint32_t ds1_lo = sdesc_lo(smem_u32(smem + OFF_DS1)), ds2_lo = sdesc_lo(smem_u32(smem + OFF_DS2));
        const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
        constexpr uint32_t DA_MN_LBO = ((DA_BYTES / 2) >> 4) << 16;   // dA as MN-major B: 64-column atoms 8 KB apart
        const uint32_t tb = tmem_base;
        int st = 0;
        for (int i = 0; i < nq; ++i) {
          const uint32_t sp_lo = st_lo0 + st * (STAGE_BYTES >> 4);
          // e_done(i) implies that stage i was loaded and that the score MMAs reading it have completed
          if (!mbar_wait(&misc->e_done, i & 1, abort_flag, 1521, i)) break;
          tc_fence_after();
          const uint32_t first = i > 0;
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            mma_ss_lo(tb + T_DV, pc_lo + k * 2, sp_lo + ((2 * Q_BYTES) >> 4) + DA_MN_LBO - (1u << 16) + k * (2048 >> 4), IDESC_DV,
                      k > 0 ? 1u : first);
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            mma_ss_lo(tb + T_DK1, ds1_lo + k * 2, sp_lo + k * (2048 >> 4), IDESC_DK, k > 0 ? 1u : first);
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            mma_ss_lo(tb + T_DK2, ds2_lo + k * 2, sp_lo + (Q_BYTES >> 4) + k * (2048 >> 4), IDESC_DK, k > 0 ? 1u : first);
          mma_commit(&misc->o_done);
          mma_commit(&misc->empty[st]);
          if (++st == ST) st = 0;
        }
        mma_commit(&misc->acc_full);
      }
    }
  } else if (warp >= WARP_DRAIN) {
    // ---- dQ drain: warp q reads TMEM lanes [32q, 32q+32) of the dQ columns: lanes 0-15 hold rows 16q..16q+15 of the
    // dQ1 tile, lanes 16-31 the same rows of the dQ2 tile; each thread adds its row of 64 floats to the workspace.
    reg_dec<REGS_DRAIN>();
    const int q4 = warp - WARP_DRAIN;
    const uint32_t t_dq = tmem_base + (uint32_t(q4 * 32) << 16) + T_DQ;
    const int br = lane >> 4;
    const int r_in_tile = q4 * 16 + (lane & 15);
    float* acc_base = args.dq_acc + (size_t(br) * gridDim.y + bh) * size_t(args.n_pad) * HD;
    for (int i = 0; i < nq; ++i) {
      const int qrow = tile_of(i) * BQ + r_in_tile;
      float* dst = acc_base + size_t(qrow) * HD;
      if (!mbar_wait_warp(&misc->dq_full, i & 1, abort_flag, 1601, i)) break;
      tc_fence_after();
      uint32_t r[32];
      tmem_ld32(t_dq, r);
      tc_wait_ld();
      if (qrow < args.n) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          red_add_v4(dst + 4 * c, __uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]),
                     __uint_as_float(r[4 * c + 3]));
      }
      tmem_ld32(t_dq + 32, r);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&misc->dq_free);
      if (qrow < args.n) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          red_add_v4(dst + 32 + 4 * c, __uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]),
                     __uint_as_float(r[4 * c + 3]));
      }
    }
  } else {
    reg_inc<REGS_ELEM>();
    const int g = warp >> 2;                       // warpgroup: query columns [16g, 16g+16) of every tile
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tb = tmem_base + lane_base;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const float sg = load_lambda(args.lambda_ptr, args.lambda_dtype) < 0.f ? 1.f : -1.f;   // -sign(lambda)
    const bool kv_valid = kv_tile * BKV + row < args.n;    // key rows past the sequence end take no part in dQ
    // dropout: this thread owns key column kv_tile*BKV + row; a hash covers two consecutive query rows of it
    const uint32_t dkey1 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 0u) : 0u;
    const uint32_t dkey2 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 1u) : 0u;
    const uint32_t dcol2 = uint32_t(kv_tile * BKV + row) >> 1;
    const int dcol_odd = row & 1;
    const float dscale = DROP ? args.drop_scale : 1.f;
    uint8_t* const pc_row = smem + OFF_PC + row * 128;
    const int ch0 = ((g * 2) ^ (row & 7)) << 4, ch1 = ((g * 2 + 1) ^ (row & 7)) << 4;
    const f32x2 sl2_2 = pk2(sl2, sl2), sg_2 = pk2(sg, sg);
    bool ok = true;
    for (int i = 0; i < nq; ++i) {
      const int st = i % ST;
      const float4* stats = reinterpret_cast<const float4*>(smem + OFF_STAGE + st * STAGE_BYTES + 2 * Q_BYTES + DA_BYTES) + g * 16;
      const int qt = tile_of(i);
      if (!mbar_wait(&misc->s_full, i & 1, abort_flag, 1701 + g, i)) { ok = false; break; }
      tc_fence_after();
      uint32_t s1[16], s2[16], dp[16];
      tmem_ld16(tb + T_S1 + g * 16, s1);
      tmem_ld16(tb + T_S2 + g * 16, s2);
      tmem_ld16(tb + T_DP + g * 16, dp);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&misc->s_free);
      {
        // hidden positions get a score of -inf (probability 0): under the causal mask the first c0 query columns
        // of this thread's 16 (the key row sees query rows >= its own index only); every column of a key row
        // past the sequence end
        int c0 = kv_valid ? 0 : 16;
        if (args.causal) c0 = max(c0, kv_tile * BKV + row - (qt * BQ + g * 16));
        if (c0 > 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < c0) { s1[j] = 0xff800000u; s2[j] = 0xff800000u; }
        }
      }
      uint32_t pc[8], d1[8], d2[8];
      // statistics of the next DA_PF / 2 column pairs (see lds_v4): {x0, x1, y0, y1} and {z0, z1, w0, w1}, negated
      float4 sva[DA_PF / 2], svb[DA_PF / 2];
#pragma unroll
      for (int j = 0; j < DA_PF / 2; ++j) { sva[j] = lds_v4(stats + 2 * j); svb[j] = lds_v4(stats + 2 * j + 1); }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float4 sa = sva[jj % (DA_PF / 2)], sb = svb[jj % (DA_PF / 2)];
        if (jj + DA_PF / 2 < 8) {
          sva[jj % (DA_PF / 2)] = lds_v4(stats + 2 * (jj + DA_PF / 2));
          svb[jj % (DA_PF / 2)] = lds_v4(stats + 2 * (jj + DA_PF / 2) + 1);
        }
        float x10, x11, x20, x21;
        up2(fma2(pk2u(s1[2 * jj], s1[2 * jj + 1]), sl2_2, pk2(sa.x, sa.y)), x10, x11);
        up2(fma2(pk2u(s2[2 * jj], s2[2 * jj + 1]), sl2_2, pk2(sa.z, sa.w)), x20, x21);
        const float p10 = ex2(x10), p11 = ex2(x11);
        const float p20 = ex2(x20), p21 = ex2(x21);     // |lam| P2
        float pcv[2], d1v[2], d2v[2];
        if constexpr (DROP) {
          // dropped positions contribute neither to dV nor to dP; kept ones carry the factor 1/(1-p)
          const uint32_t drow2 = uint32_t(qt * (BQ / 2) + g * 8 + jj);
          const uint32_t h1 = drop_hash(dkey1, drow2, dcol2), h2 = drop_hash(dkey2, drow2, dcol2);
          const float p1v[2] = {p10, p11}, p2v[2] = {p20, p21};
          const float nz[2] = {sb.x, sb.y}, nw[2] = {sb.z, sb.w};
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float dpv = __uint_as_float(dp[2 * jj + u]);
            const float k1 = drop_keep(h1, 2 * u + dcol_odd, args.drop_thresh) ? dscale : 0.f;
            const float k2 = drop_keep(h2, 2 * u + dcol_odd, args.drop_thresh) ? sg * dscale : 0.f;
            pcv[u] = fmaf(k2, p2v[u], k1 * p1v[u]);
            d1v[u] = p1v[u] * fmaf(k1, dpv, nz[u]);
            d2v[u] = p2v[u] * fmaf(k2, dpv, nw[u]);
          }
        } else {
          const f32x2 p1_2 = pk2(p10, p11), p2_2 = pk2(p20, p21), dp_2 = pk2u(dp[2 * jj], dp[2 * jj + 1]);
          up2(fma2(sg_2, p2_2, p1_2), pcv[0], pcv[1]);
          up2(mul2(p1_2, add2(dp_2, pk2(sb.x, sb.y))), d1v[0], d1v[1]);
          up2(mul2(p2_2, fma2(sg_2, dp_2, pk2(sb.z, sb.w))), d2v[0], d2v[1]);
        }
        pc[jj] = pack2<BF>(pcv[0], pcv[1]);
        d1[jj] = pack2<BF>(d1v[0], d1v[1]);
        d2[jj] = pack2<BF>(d2v[0], d2v[1]);
      }
      // the shared-memory tiles of tile i-1 (Pc, dS1^T, dS2^T) must have been consumed by its dV, dK and dQ MMAs
      if (i > 0) {
        if (!mbar_wait(&misc->o_done, (i - 1) & 1, abort_flag, 1709 + g, i)) { ok = false; break; }
      }
      // Pc, dS1^T, dS2^T tiles [128 key rows][64 query columns], 128-byte rows, 16-byte chunks XOR-swizzled by row
      *reinterpret_cast<uint4*>(pc_row + ch0) = make_uint4(pc[0], pc[1], pc[2], pc[3]);
      *reinterpret_cast<uint4*>(pc_row + ch1) = make_uint4(pc[4], pc[5], pc[6], pc[7]);
      *reinterpret_cast<uint4*>(pc_row + (OFF_DS1 - OFF_PC) + ch0) = make_uint4(d1[0], d1[1], d1[2], d1[3]);
      *reinterpret_cast<uint4*>(pc_row + (OFF_DS1 - OFF_PC) + ch1) = make_uint4(d1[4], d1[5], d1[6], d1[7]);
      *reinterpret_cast<uint4*>(pc_row + (OFF_DS2 - OFF_PC) + ch0) = make_uint4(d2[0], d2[1], d2[2], d2[3]);
      *reinterpret_cast<uint4*>(pc_row + (OFF_DS2 - OFF_PC) + ch1) = make_uint4(d2[4], d2[5], d2[6], d2[7]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&misc->e_done);
    }
    ok = ok && mbar_wait(&misc->acc_full, 0, abort_flag, 1711 + g);
    tc_fence_after();
    // warpgroup g reads accumulator columns [64g, 64g+64): g = 0,1 -> the two halves of dV, g = 2 -> dK1, g = 3 -> dK2.
    // The gradients leave through shared memory and the TMA engine: each warpgroup lays its 64 columns into a
    // swizzled [128][64] tile over the resident K1 / K2 / V tiles, which no MMA reads any more (acc_full follows
    // the last dQ MMAs), and one of its threads stores the tile.  The engine clips at the tensor's bounds.
    {
      const float s = g < 2 ? 1.f : args.sm_scale;
      uint8_t* tile = smem + ((g + 2) & 3) * K_BYTES;     // g = 0,1 -> the two halves of V; 2 -> K1; 3 -> K2
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t acc[32];
        tmem_ld32(tb + g * 64 + h * 32, acc);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack2<BF>(__uint_as_float(acc[8 * c + 0]) * s, __uint_as_float(acc[8 * c + 1]) * s);
          v.y = pack2<BF>(__uint_as_float(acc[8 * c + 2]) * s, __uint_as_float(acc[8 * c + 3]) * s);
          v.z = pack2<BF>(__uint_as_float(acc[8 * c + 4]) * s, __uint_as_float(acc[8 * c + 5]) * s);
          v.w = pack2<BF>(__uint_as_float(acc[8 * c + 6]) * s, __uint_as_float(acc[8 * c + 7]) * s);
          st_swizzled_chunk(tile, row, h * 4 + c, v);
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1 + g, 128);
      const int dv_real = 2 * args.d;
      if ((warp & 3) == 0 && elect_one()) {
        if (ok && !*abort_flag && (g != 1 || dv_real > 64)) {
          const CUtensorMap* map = g < 2 ? &tm_dv : (g == 2 ? &tm_dk1 : &tm_dk2);
          tma_store_4d(tile, map, g == 1 ? 64 : 0, kv_tile * BKV, bh, 0);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_S) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dQ_b = sm_scale * (sum of the key blocks' partial sums), fp32 -> 16 bit.  One thread = 8 columns of one row.
template <bool BF>
__global__ void __launch_bounds__(256) diffattn_bwd_dq_finish_kernel(const BwdArgs args, int bh_total) {
  const int d8 = args.d >> 3;                                   // 16-byte pieces per output row
  const long long per_branch = (long long)bh_total * args.n * d8;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < 2 * per_branch; t += (long long)gridDim.x * blockDim.x) {
    const int br = t >= per_branch;
    const long long u = t - br * per_branch;
    const int c = int(u % d8);
    const long long rowg = u / d8;                              // bh * n + row
    const long long bh_i = rowg / args.n;
    const long long row = rowg - bh_i * args.n;
    const float4* src = reinterpret_cast<const float4*>(args.dq_acc + ((size_t(br) * bh_total + bh_i) * args.n_pad + row) * 64 + c * 8);
    const float4 a = src[0], b = src[1];
    const float s = args.sm_scale;
    uint4 v;
    v.x = pack2<BF>(a.x * s, a.y * s); v.y = pack2<BF>(a.z * s, a.w * s);
    v.z = pack2<BF>(b.x * s, b.y * s); v.w = pack2<BF>(b.z * s, b.w * s);
    *reinterpret_cast<uint4*>((br ? args.dq2 : args.dq1) + rowg * args.d + c * 8) = v;
  }
}

}  // namespace da
