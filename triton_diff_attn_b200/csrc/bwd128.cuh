// Differential-attention backward for head dim D = 128 (value width 256), sm_100a.
//
// At this width the accumulators of the D = 64 design (dV, dK1, dK2 in one CTA) need all 512 TMEM
// columns, so the work is cut differently (same math as src/kernel.py:410-436 of the reference):
//   * diffattn_bwd_side128_kernel<QSIDE>  one branch b per CTA (blockIdx.z).  With X the stationary
//       operand of the branch and Z the streamed one:  S = X Z^T,  T = Y W^T,  dS = +-P (T - E),
//       OUT += dS Z.   QSIDE:  X = Q_b, Y = dA, Z = K_b, W = V   -> OUT = dQ_b  (thread = query row)
//                      !QSIDE: X = K_b, Y = V,  Z = Q_b, W = dA  -> OUT = dK_b  (thread = key row; S, T transposed)
//   * diffattn_bwd_dv128_kernel           dV += (P1 - lam P2)^T dA, key/value-stationary, both branches.
// TMEM and shared-memory conventions are those of bwd.cuh; streamed tiles are 64 rows.
#pragma once
#include "bwd.cuh"
#include "sm100.cuh"

namespace da {

namespace side128 {
// Two rings for the streamed operands, because their lifetimes differ: W feeds only the T scores and is free as soon
// as those MMAs have completed; Z feeds the S scores AND the output MMAs of its sub-tile, one elementwise pass
// later.  With one ring of {Z, W} stages the next load could only be requested after the output MMAs, and its whole
// latency sat between two sub-tiles (the kernel ran at half the tensor pipe's pace).
constexpr int BM = 128, SUB = 64, HD = 128, DV = 256, ZST = 4, WST = 3, NWG = 4;
constexpr int X_BYTES = BM * HD * 2;        // 32 KB: two boxes [128 x 64]
constexpr int Y_BYTES = BM * DV * 2;        // 64 KB: four boxes [128 x 64]
constexpr int Z_BYTES = SUB * HD * 2;       // 16 KB: two boxes [64 x 64]
constexpr int W_BYTES = SUB * DV * 2;       // 32 KB: four boxes [64 x 64]
constexpr int STAT_BYTES = SUB * 16;        // 1 KB
constexpr int ZSTAGE_BYTES = Z_BYTES + STAT_BYTES;            // 17 KB: the per-column statistics travel with Z
constexpr int OFF_X = 0, OFF_Y = X_BYTES, OFF_W = X_BYTES + Y_BYTES;       // 96 KB
constexpr int OFF_Z = OFF_W + 2 * W_BYTES;                                 // 160 KB
// Once Y has been copied into TMEM its 64 KB tile is ring space: the W ring has three stages (its own two and the
// first half of Y's tile), the Z ring four (its own three and one in the second half of Y's tile).  The stages in
// Y's tile are first filled for sub-tiles 2 (W) and 3 (Z), after the copy.
static_assert(WST == 3 && ZST == 4 && Y_BYTES == 2 * W_BYTES && ZSTAGE_BYTES <= W_BYTES, "ring stages inside the Y tile");
__host__ __device__ constexpr int w_stage_off(int s) { return OFF_Y + ((s + 2) & 3) * W_BYTES; }
__host__ __device__ constexpr int z_stage_off(int s) { return s < 3 ? OFF_Z + s * ZSTAGE_BYTES : OFF_Y + W_BYTES; }
constexpr int OFF_MISC = OFF_Z + 3 * ZSTAGE_BYTES;                       // 211 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int NUM_THREADS = NWG * 128 + 64;
constexpr int WARP_TMA = NWG * 4, WARP_MMA = NWG * 4 + 1;
// TMEM: S two 64-column buffers [0,128) | T likewise [128,256) | OUT [256,384) | Y as 16-bit pairs [384,512).
// Y (the stationary 256-wide operand) is copied from its shared-memory tile into TMEM once per CTA and serves as the
// TMEM A operand of T = Y W^T: those 16 MMAs per sub-tile then read only W from shared memory (2 KB instead of 6 KB
// per step), which is what bounds this kernel.
constexpr int T_S = 0, T_T = 128, T_OUT = 256, T_Y = 384;
struct Misc {
  uint64_t bar_xy, y_ready;
  uint64_t full[WST], zempty[ZST], wempty[WST];
  uint64_t s_full[2], ds_full[2], acc_full;
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace side128

// tm_x, tm_z: the branch's stationary / streamed [N, 128] operand (box rows 128 / 64);
// tm_y, tm_w: the [N, 256] operands.  dA lives in the dense workspace and is addressed (col, row, b*h, 0).
template <bool QSIDE, bool BF, bool DROP>
__global__ void __launch_bounds__(side128::NUM_THREADS, 1)
diffattn_bwd_side128_kernel(const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
                            const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_z0,
                            const __grid_constant__ CUtensorMap tm_z1, const __grid_constant__ CUtensorMap tm_w,
                            const BwdArgs args) {
  using namespace side128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal, query side: the later a query tile, the more keys it sees -- the heaviest tiles are launched first (on the key
  // side the first key tiles are the heaviest already)
  const int tile = (QSIDE && args.causal) ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x), bh = blockIdx.y, br = blockIdx.z;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  // streamed 64-row sub-tiles t0 .. t0+nsub-1 (local index t).  Causal: the query side streams keys up to its
  // diagonal tile, the key side streams queries from its diagonal tile on.
  const int nsub_all = args.n_pad / SUB;
  const int t0 = (args.causal && !QSIDE) ? 2 * tile : 0;
  const int nsub = (args.causal && QSIDE) ? min(nsub_all, 2 * (tile + 1)) : nsub_all - t0;
  const CUtensorMap* tm_x = br ? &tm_x1 : &tm_x0;
  const CUtensorMap* tm_z = br ? &tm_z1 : &tm_z0;
  // dA is the Y operand on the query side and the W operand on the key side
  const int y_c2 = QSIDE ? bh : h_idx, y_c3 = QSIDE ? 0 : b_idx;
  const int w_c2 = QSIDE ? h_idx : bh, w_c3 = QSIDE ? b_idx : 0;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_xy, 1);
    mbar_init(&misc->y_ready, NWG * 128);
    for (int i = 0; i < ZST; ++i) mbar_init(&misc->zempty[i], 1);
    for (int i = 0; i < WST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->wempty[i], 1); }
    for (int u = 0; u < 2; ++u) { mbar_init(&misc->s_full[u], 1); mbar_init(&misc->ds_full[u], NWG * 128); }
    mbar_init(&misc->acc_full, 1);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == WARP_MMA) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    if (elect_one()) {
      mbar_expect_tx(&misc->bar_xy, X_BYTES + Y_BYTES);
      for (int c = 0; c < 2; ++c) tma_load_4d(smem + OFF_X + c * 16384, tm_x, &misc->bar_xy, c * 64, tile * BM, h_idx, b_idx);
      for (int c = 0; c < 4; ++c) tma_load_4d(smem + OFF_Y + c * 16384, &tm_y, &misc->bar_xy, c * 64, tile * BM, y_c2, y_c3);
      int zs = 0, ws = 0;
      uint32_t zpar = 1, wpar = 1;
      for (int t = 0; t < nsub; ++t) {
        uint8_t* zp = smem + z_stage_off(zs);
        uint8_t* wp = smem + w_stage_off(ws);
        if (t == 2 && !mbar_wait(&misc->y_ready, 0, abort_flag, 1103, t)) break;     // stage 2 is Y's tile
        if (!mbar_wait(&misc->zempty[zs], zpar, abort_flag, 1101, t)) break;
        if (!mbar_wait(&misc->wempty[ws], wpar, abort_flag, 1102, t)) break;
        // one arrival barrier per sub-tile for both operands (indexed like the W ring, the shallower one): the issuer
        // pays one wait instead of two -- every mbarrier wait costs it 110-150 clocks even when the phase is complete
        mbar_expect_tx(&misc->full[ws], (QSIDE ? Z_BYTES : ZSTAGE_BYTES) + W_BYTES);
        for (int c = 0; c < 2; ++c) tma_load_4d(zp + c * 8192, tm_z, &misc->full[ws], c * 64, (t0 + t) * SUB, h_idx, b_idx);
        if (!QSIDE)
          bulk_load_1d(zp + Z_BYTES, args.stats + (size_t(bh) * args.n_pad + size_t(t0 + t) * SUB), STAT_BYTES, &misc->full[ws]);
        for (int c = 0; c < 4; ++c) tma_load_4d(wp + c * 8192, &tm_w, &misc->full[ws], c * 64, (t0 + t) * SUB, w_c2, w_c3);
        if (++zs == ZST) { zs = 0; zpar ^= 1; }
        if (++ws == WST) { ws = 0; wpar ^= 1; }
      }
    }
  } else if (warp == WARP_MMA) {
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);
      constexpr uint32_t IDESC_OUT = make_idesc(BM, HD, 0, 1, BF);     // OUT += dS Z, Z MN-major (two 64-column atoms)
      const uint32_t x_lo = sdesc_lo(smem_u32(smem + OFF_X));
      const uint32_t s_lo0 = sdesc_lo(smem_u32(smem)), w_lo0 = sdesc_lo(smem_u32(smem + OFF_Y));
      const uint32_t tb = tmem_base;
      // scores of one sub-tile: S from the Z stage zs, T from the W stage ws; W is free once these MMAs have completed
      auto issue_scores = [&](int zs, int ws, int u) {
        const uint32_t z_lo = s_lo0 + (z_stage_off(zs) >> 4), w_lo = w_lo0 + ((ws + 2) & 3) * (W_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ss_lo(tb + T_S + u * SUB, x_lo + (k / 4) * (16384 >> 4) + (k % 4) * 2, z_lo + (k / 4) * (8192 >> 4) + (k % 4) * 2,
                    IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)
          mma_ts_lo(tb + T_T + u * SUB, tb + T_Y + k * 8, w_lo + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[u]);
        mma_commit(&misc->wempty[ws]);
      };
      bool ok = mbar_wait(&misc->bar_xy, 0, abort_flag, 1201);
      ok = ok && mbar_wait(&misc->y_ready, 0, abort_flag, 1206);
      ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 1202);
      if (ok) {
        tc_fence_after();
        issue_scores(0, 0, 0);
        int zs = 0, ws = 0;                 // stages of sub-tile t
        uint32_t wpar = 0;
        for (int t = 0; t < nsub; ++t) {
          const int u = t & 1;
          const uint32_t sp_lo = s_lo0 + (z_stage_off(zs) >> 4);
          int zs_n = zs + 1, ws_n = ws + 1;
          uint32_t wpar_n = wpar;
          if (zs_n == ZST) zs_n = 0;
          if (ws_n == WST) { ws_n = 0; wpar_n ^= 1; }
          if (t + 1 < nsub) {
            if (!mbar_wait(&misc->full[ws_n], wpar_n, abort_flag, 1203, t)) break;
            tc_fence_after();
            issue_scores(zs_n, ws_n, u ^ 1);
          }
          if (!mbar_wait(&misc->ds_full[u], (t >> 1) & 1, abort_flag, 1204, t)) break;
          tc_fence_after();
          // Z as MN-major B: N = 128 columns = two atoms 8 KB apart, K = the 64 streamed rows
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(tb + T_OUT, tb + T_S + u * SUB + k * 16, sp_lo + ((8192u >> 4) << 16) - (1u << 16) + k * (2048 >> 4), IDESC_OUT,
                      (t > 0 || k > 0));
          mma_commit(&misc->zempty[zs]);
          zs = zs_n;
          ws = ws_n; wpar = wpar_n;
        }
        mma_commit(&misc->acc_full);
      }
    }
  } else {
    const int g = warp >> 2;                       // columns [16g, 16g+16) of every sub-tile
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tb = tmem_base + lane_base;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
    const float sg = (br && !(lam < 0.f)) ? -1.f : 1.f;      // branch 2: -sign(lambda); |lambda| is in the statistics
    const size_t grow = size_t(bh) * args.n + size_t(tile) * BM + row;
    float neg_l = 0.f, neg_e = 0.f;        // the statistics are stored negated (BwdArgs::stats)
    if (QSIDE) {
      const float4 sv = stat_row(args.stats, size_t(bh) * args.n_pad + size_t(tile) * BM + row);
      neg_l = br ? sv.y : sv.x;
      neg_e = br ? sv.w : sv.z;
    }
    const f32x2 sl2_2 = pk2(sl2, sl2), sg_2 = pk2(sg, sg);
    // dropout: `own` is this thread's fixed coordinate (query row on the query side, key column on the key side)
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t down2 = uint32_t(tile * BM + row) >> 1;
    const int down_odd = row & 1;
    const float sgs = DROP ? sg * args.drop_scale : sg;
    bool ok = mbar_wait(&misc->bar_xy, 0, abort_flag, 1300 + g);
    {
      // Y into TMEM: this thread's row, the 64 columns of box g (128 bytes, swizzled in 16-byte chunks) -> 32 columns
      uint32_t yv[32];
      const uint8_t* yrow = smem + OFF_Y + g * 16384 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(yrow + ((c ^ (row & 7)) << 4));
        yv[4 * c] = v.x; yv[4 * c + 1] = v.y; yv[4 * c + 2] = v.z; yv[4 * c + 3] = v.w;
      }
      tmem_st32(tb + T_Y + g * 32, yv);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->y_ready);
    }
    int st = 0;
    for (int t = 0; ok && t < nsub; ++t) {
      const int u = t & 1;
      const uint32_t t_s = tb + T_S + u * SUB + g * 16, t_t = tb + T_T + u * SUB + g * 16;
      const float4* stats = reinterpret_cast<const float4*>(smem + z_stage_off(st) + Z_BYTES) + g * 16;
      if (!mbar_wait(&misc->s_full[u], (t >> 1) & 1, abort_flag, 1301 + g, t)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[16], tt[16], ds[8];
      tmem_ld16(t_s, s);
      tmem_ld16(t_t, tt);
      tc_wait_ld();
      if (QSIDE) {
        // query side: streamed columns are key rows; those >= N, or (causal) right of this row's diagonal, get
        // probability 0.  (On the key side the streamed columns are query rows: out-of-range ones already have
        // neutral statistics, and the causal mask hides the columns LEFT of the diagonal.)
        const int c_first = t * SUB + g * 16;
        int nv = args.n - c_first;
        if (args.causal) nv = min(nv, tile * BM + row - c_first + 1);
        if (nv < 16) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i >= nv) s[i] = 0xff800000u;
        }
      } else if (args.causal) {
        const int c0 = tile * BM + row - ((t0 + t) * SUB + g * 16);
        if (c0 > 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < c0) s[i] = 0xff800000u;
        }
      }
      // key side: statistics of the next DA_PF / 2 pairs of streamed columns, {x0, x1, y0, y1} and {z0, z1, w0, w1}
      float4 sva[DA_PF / 2], svb[DA_PF / 2];
      if (!QSIDE) {
#pragma unroll
        for (int j = 0; j < DA_PF / 2; ++j) { sva[j] = lds_v4(stats + 2 * j); svb[j] = lds_v4(stats + 2 * j + 1); }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f32x2 nl_2 = pk2(neg_l, neg_l), ne_2 = pk2(neg_e, neg_e);
        if (!QSIDE) {
          const float4 sa = sva[i % (DA_PF / 2)], sb = svb[i % (DA_PF / 2)];
          if (i + DA_PF / 2 < 8) {
            sva[i % (DA_PF / 2)] = lds_v4(stats + 2 * (i + DA_PF / 2));
            svb[i % (DA_PF / 2)] = lds_v4(stats + 2 * (i + DA_PF / 2) + 1);
          }
          nl_2 = br ? pk2(sa.z, sa.w) : pk2(sa.x, sa.y);
          ne_2 = br ? pk2(sb.z, sb.w) : pk2(sb.x, sb.y);
        }
        float x0, x1, v0, v1;
        up2(fma2(pk2u(s[2 * i], s[2 * i + 1]), sl2_2, nl_2), x0, x1);
        const f32x2 p_2 = pk2(ex2(x0), ex2(x1));
        f32x2 sge_2 = sg_2;
        if constexpr (DROP) {
          // streamed index of this pair: key columns on the query side, query rows on the key side
          const uint32_t str2 = uint32_t((QSIDE ? t : t0 + t) * (SUB / 2) + g * 8 + i);
          const uint32_t hh = QSIDE ? drop_hash(dkey, down2, str2) : drop_hash(dkey, str2, down2);
          sge_2 = pk2(drop_keep(hh, QSIDE ? 2 * down_odd : down_odd, args.drop_thresh) ? sgs : 0.f,
                      drop_keep(hh, QSIDE ? 2 * down_odd + 1 : 2 + down_odd, args.drop_thresh) ? sgs : 0.f);
        }
        up2(mul2(p_2, fma2(sge_2, pk2u(tt[2 * i], tt[2 * i + 1]), ne_2)), v0, v1);
        ds[i] = pack2<BF>(v0, v1);
      }
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                   ::"r"(t_s), "r"(ds[0]), "r"(ds[1]), "r"(ds[2]), "r"(ds[3]), "r"(ds[4]), "r"(ds[5]), "r"(ds[6]), "r"(ds[7]) : "memory");
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->ds_full[u]);
      if (++st == ZST) st = 0;
    }
    ok = ok && mbar_wait(&misc->acc_full, 0, abort_flag, 1311 + g);
    tc_fence_after();
    uint32_t acc[32];
    tmem_ld32(tb + T_OUT + g * 32, acc);
    tc_wait_ld();
    if (ok && !*abort_flag && tile * BM + row < args.n) {
      const float sc = args.sm_scale;
      __half* out = QSIDE ? (br ? args.dq2 : args.dq1) : (br ? args.dk2 : args.dk1);
      uint4* p = reinterpret_cast<uint4*>(out + grow * HD + g * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 v;
        v.x = pack2<BF>(__uint_as_float(acc[8 * i + 0]) * sc, __uint_as_float(acc[8 * i + 1]) * sc);
        v.y = pack2<BF>(__uint_as_float(acc[8 * i + 2]) * sc, __uint_as_float(acc[8 * i + 3]) * sc);
        v.z = pack2<BF>(__uint_as_float(acc[8 * i + 4]) * sc, __uint_as_float(acc[8 * i + 5]) * sc);
        v.w = pack2<BF>(__uint_as_float(acc[8 * i + 6]) * sc, __uint_as_float(acc[8 * i + 7]) * sc);
        p[i] = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dV for D = 128: one CTA = 128 key/value rows; query tiles of 64 rows stream by.
// TMEM: dV [0,256) | S1^T [256,320) | S2^T [320,384) | K1 as 16-bit pairs [384,448) | K2 [448,512).
// K1 and K2 are copied once per CTA from their shared-memory tiles into TMEM and serve as the TMEM A operands of
// S_b^T = K_b Q_b^T (those MMAs then read only Q_b from shared memory); their 64 KB then hold the two buffers of
// (P1 - lam P2)^T (K-major A operand of dV += Pc^T dA) and a third stage of the Q ring.  With two Pc buffers a
// warpgroup never waits for the dV MMAs of the tile before; the scores are single-buffered (the next tile's are issued
// as soon as this tile's are in registers).
// ------------------------------------------------------------------------------------------------
namespace dv128 {
// Three rings, by lifetime: {Q1, Q2} feed the score MMAs and are free once those have completed; the per-column
// statistics (1 KB) are read by the warpgroups until the end of their pass; dA feeds the dV MMAs after that pass.
constexpr int BKV = 128, BQ = 64, HD = 128, DV = 256, QST = 3, AST = 2, TST = 4, NWG = 4;
constexpr int K_BYTES = BKV * HD * 2;       // 32 KB: two boxes [128 x 64]
constexpr int Q_BYTES = BQ * HD * 2;        // 16 KB: two boxes [64 x 64]
constexpr int DA_BYTES = BQ * DV * 2;       // 32 KB: four boxes [64 x 64]
constexpr int STAT_BYTES = BQ * 16;
constexpr int QSTAGE_BYTES = 2 * Q_BYTES;                          // 32 KB
constexpr int PC_BYTES = BKV * BQ * 2;      // 16 KB
constexpr int OFF_K1 = 0, OFF_K2 = K_BYTES, OFF_QS = 2 * K_BYTES;                                  // 64 KB
constexpr int OFF_DA = OFF_QS + 2 * QSTAGE_BYTES;                                                  // 128 KB
constexpr int OFF_ST = OFF_DA + AST * DA_BYTES;                                                    // 192 KB
constexpr int OFF_MISC = OFF_ST + TST * STAT_BYTES;                                                // 196 KB
// after the copy of K1, K2 into TMEM: Pc buffer b at OFF_PC + b * PC_BYTES, Q stage 2 in the second half of the K tiles
constexpr int OFF_PC = 0;
static_assert(QST == 3 && 2 * PC_BYTES + QSTAGE_BYTES <= 2 * K_BYTES, "Pc buffers and the third Q stage live in the K tiles");
__host__ __device__ constexpr int q_stage_off(int s) { return s < 2 ? OFF_QS + s * QSTAGE_BYTES : 2 * PC_BYTES; }
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int NUM_THREADS = NWG * 128 + 64;
constexpr int WARP_TMA = NWG * 4, WARP_MMA = NWG * 4 + 1;
constexpr int T_DV = 0, T_S1 = 256, T_S2 = 320, T_K1 = 384, T_K2 = 448;
struct Misc {
  uint64_t bar_kv, k_ready;
  uint64_t qfull[QST], qempty[QST], afull[AST], aempty[AST], tempty[TST];
  uint64_t s_full, s_free, e_done, mma_done[2], acc_full;
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace dv128

template <bool BF, bool DROP>
__global__ void __launch_bounds__(dv128::NUM_THREADS, 1)
diffattn_bwd_dv128_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                          const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                          const __grid_constant__ CUtensorMap tm_da, const BwdArgs args) {
  using namespace dv128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, bh = blockIdx.y;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  const int nq_all = args.n_pad / BQ;
  const int i0 = args.causal ? kv_tile * (BKV / BQ) : 0;     // causal: query tiles from the diagonal on
  const int nq = nq_all - i0;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_kv, 1);
    for (int i = 0; i < QST; ++i) { mbar_init(&misc->qfull[i], 1); mbar_init(&misc->qempty[i], 1); }
    for (int i = 0; i < TST; ++i) mbar_init(&misc->tempty[i], 1);
    for (int i = 0; i < AST; ++i) { mbar_init(&misc->afull[i], 1); mbar_init(&misc->aempty[i], 1); }
    mbar_init(&misc->k_ready, NWG * 128);
    mbar_init(&misc->s_full, 1);
    mbar_init(&misc->s_free, NWG * 128);
    mbar_init(&misc->e_done, NWG * 128);
    for (int u = 0; u < 2; ++u) mbar_init(&misc->mma_done[u], 1);
    mbar_init(&misc->acc_full, 1);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == WARP_MMA) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    if (elect_one()) {
      mbar_expect_tx(&misc->bar_kv, 2 * K_BYTES);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(smem + OFF_K1 + c * 16384, &tm_k1, &misc->bar_kv, c * 64, kv_tile * BKV, h_idx, b_idx);
        tma_load_4d(smem + OFF_K2 + c * 16384, &tm_k2, &misc->bar_kv, c * 64, kv_tile * BKV, h_idx, b_idx);
      }
      int qs = 0, as = 0, ts = 0;
      uint32_t qpar = 1, apar = 1, tpar = 1;
      for (int i = 0; i < nq; ++i) {
        uint8_t* qp = smem + q_stage_off(qs);
        uint8_t* ap = smem + OFF_DA + as * DA_BYTES;
        if (i == 2 && !mbar_wait(&misc->k_ready, 0, abort_flag, 1404, i)) break;      // Q stage 2 lies in the K tiles
        // Q1, Q2 and the statistics of a tile arrive on ONE barrier (the Q ring's): every mbarrier wait costs the issuer
        // 100-150 clocks even when the phase is complete
        if (!mbar_wait(&misc->qempty[qs], qpar, abort_flag, 1401, i)) break;
        if (!mbar_wait(&misc->tempty[ts], tpar, abort_flag, 1403, i)) break;
        mbar_expect_tx(&misc->qfull[qs], QSTAGE_BYTES + STAT_BYTES);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(qp + c * 8192, &tm_q1, &misc->qfull[qs], c * 64, (i0 + i) * BQ, h_idx, b_idx);
          tma_load_4d(qp + Q_BYTES + c * 8192, &tm_q2, &misc->qfull[qs], c * 64, (i0 + i) * BQ, h_idx, b_idx);
        }
        bulk_load_1d(smem + OFF_ST + ts * STAT_BYTES, args.stats + (size_t(bh) * args.n_pad + size_t(i0 + i) * BQ), STAT_BYTES, &misc->qfull[qs]);
        if (!mbar_wait(&misc->aempty[as], apar, abort_flag, 1402, i)) break;
        mbar_expect_tx(&misc->afull[as], DA_BYTES);
        for (int c = 0; c < 4; ++c) tma_load_4d(ap + c * 8192, &tm_da, &misc->afull[as], c * 64, (i0 + i) * BQ, bh, 0);
        if (++qs == QST) { qs = 0; qpar ^= 1; }
        if (++as == AST) { as = 0; apar ^= 1; }
        if (++ts == TST) { ts = 0; tpar ^= 1; }
      }
    }
  } else if (warp == WARP_MMA) {
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BKV, BQ, 0, 0, BF);
      constexpr uint32_t IDESC_DV = make_idesc(BKV, DV, 0, 1, BF);     // N = 256: dA as MN-major B, four atoms 8 KB apart
      const uint32_t s_lo0 = sdesc_lo(smem_u32(smem));
      const uint32_t a_lo0 = sdesc_lo(smem_u32(smem + OFF_DA));
      const uint32_t tb = tmem_base;
      // scores of a tile from Q stage qs; Q is free once these MMAs have completed
      auto issue_scores = [&](int qs) {
        const uint32_t sp_lo = s_lo0 + (q_stage_off(qs) >> 4);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ts_lo(tb + T_S1, tb + T_K1 + k * 8, sp_lo + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ts_lo(tb + T_S2, tb + T_K2 + k * 8, sp_lo + (Q_BYTES >> 4) + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full);             // (the statistics of the tile arrived with Q: s_full implies them)
        mma_commit(&misc->qempty[qs]);
      };
      bool ok = mbar_wait(&misc->k_ready, 0, abort_flag, 1501);
      ok = ok && mbar_wait(&misc->qfull[0], 0, abort_flag, 1502);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
        int qs = 0, as = 0, ts = 0;
        uint32_t qpar = 0, apar = 0;
        for (int i = 0; i < nq; ++i) {
          int qs_n = qs + 1;
          uint32_t qpar_n = qpar;
          if (qs_n == QST) { qs_n = 0; qpar_n ^= 1; }
          if (i + 1 < nq) {
            if (!mbar_wait(&misc->qfull[qs_n], qpar_n, abort_flag, 1503, i)) break;
            if (!mbar_wait(&misc->s_free, i & 1, abort_flag, 1506, i)) break;       // the scores of tile i are in registers
            tc_fence_after();
            issue_scores(qs_n);
          }
          if (!mbar_wait(&misc->afull[as], apar, abort_flag, 1505, i)) break;     // long loaded: waited for under the warpgroups' pass
          if (!mbar_wait(&misc->e_done, i & 1, abort_flag, 1504, i)) break;
          tc_fence_after();
          mbar_arrive(&misc->tempty[ts]);        // the warpgroups have read the statistics of tile i (plain arrival)
          const uint32_t pc_lo = s_lo0 + ((OFF_PC + (i & 1) * PC_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            mma_ss_lo(tb + T_DV, pc_lo + k * 2, a_lo0 + as * (DA_BYTES >> 4) + ((8192u >> 4) << 16) - (1u << 16) + k * (2048 >> 4),
                      IDESC_DV, (i > 0 || k > 0));
          mma_commit(&misc->mma_done[i & 1]);
          mma_commit(&misc->aempty[as]);
          qs = qs_n; qpar = qpar_n;
          if (++ts == TST) ts = 0;
          if (++as == AST) { as = 0; apar ^= 1; }
        }
        mma_commit(&misc->acc_full);
      }
    }
  } else {
    const int g = warp >> 2;                       // query columns [16g, 16g+16) of every tile
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tb = tmem_base + lane_base;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const float sg = load_lambda(args.lambda_ptr, args.lambda_dtype) < 0.f ? 1.f : -1.f;   // -sign(lambda)
    const uint32_t dkey1 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 0u) : 0u;
    const uint32_t dkey2 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 1u) : 0u;
    const uint32_t dcol2 = uint32_t(kv_tile * BKV + row) >> 1;
    const int dcol_odd = row & 1;
    const f32x2 sl2_2 = pk2(sl2, sl2), sg_2 = pk2(sg, sg);
    bool ok = mbar_wait(&misc->bar_kv, 0, abort_flag, 1600 + g);
    {
      // K1, K2 into TMEM: this thread's row, the 64 columns of box g (K1 low, K1 high, K2 low, K2 high: 128 bytes,
      // swizzled in 16-byte chunks) -> 32 columns
      uint32_t kv[32];
      const uint8_t* krow = smem + OFF_K1 + g * 16384 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(krow + ((c ^ (row & 7)) << 4));
        kv[4 * c] = v.x; kv[4 * c + 1] = v.y; kv[4 * c + 2] = v.z; kv[4 * c + 3] = v.w;
      }
      tmem_st32(tb + T_K1 + g * 32, kv);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->k_ready);
    }
    int st = 0;
    for (int i = 0; ok && i < nq; ++i) {
      const float4* stats = reinterpret_cast<const float4*>(smem + OFF_ST + st * STAT_BYTES) + g * 16;
      if (!mbar_wait(&misc->s_full, i & 1, abort_flag, 1601 + g, i)) { ok = false; break; }
      tc_fence_after();
      uint32_t s1[16], s2[16], pc[8];
      tmem_ld16(tb + T_S1 + g * 16, s1);
      tmem_ld16(tb + T_S2 + g * 16, s2);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&misc->s_free);
      if (args.causal) {
        const int c0 = kv_tile * BKV + row - ((i0 + i) * BQ + g * 16);   // hidden query columns left of the diagonal
        if (c0 > 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (j < c0) { s1[j] = 0xff800000u; s2[j] = 0xff800000u; }
        }
      }
      // {x0, x1, y0, y1} (negated) of the next DA_PF / 2 column pairs (see lds_v4 in bwd.cuh)
      float4 sva[DA_PF / 2];
#pragma unroll
      for (int j = 0; j < DA_PF / 2; ++j) sva[j] = lds_v4(stats + 2 * j);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float4 sa = sva[jj % (DA_PF / 2)];
        if (jj + DA_PF / 2 < 8) sva[jj % (DA_PF / 2)] = lds_v4(stats + 2 * (jj + DA_PF / 2));
        float x10, x11, x20, x21, v0, v1;
        up2(fma2(pk2u(s1[2 * jj], s1[2 * jj + 1]), sl2_2, pk2(sa.x, sa.y)), x10, x11);
        up2(fma2(pk2u(s2[2 * jj], s2[2 * jj + 1]), sl2_2, pk2(sa.z, sa.w)), x20, x21);
        const f32x2 p1_2 = pk2(ex2(x10), ex2(x11)), p2_2 = pk2(ex2(x20), ex2(x21));
        if constexpr (DROP) {
          const uint32_t drow2 = uint32_t((i0 + i) * (BQ / 2) + g * 8 + jj);
          const uint32_t h1 = drop_hash(dkey1, drow2, dcol2), h2 = drop_hash(dkey2, drow2, dcol2);
          const float ds1 = args.drop_scale, ds2 = sg * args.drop_scale;
          const f32x2 k1_2 = pk2(drop_keep(h1, dcol_odd, args.drop_thresh) ? ds1 : 0.f, drop_keep(h1, 2 + dcol_odd, args.drop_thresh) ? ds1 : 0.f);
          const f32x2 k2_2 = pk2(drop_keep(h2, dcol_odd, args.drop_thresh) ? ds2 : 0.f, drop_keep(h2, 2 + dcol_odd, args.drop_thresh) ? ds2 : 0.f);
          up2(fma2(k2_2, p2_2, mul2(k1_2, p1_2)), v0, v1);
        } else {
          up2(fma2(sg_2, p2_2, p1_2), v0, v1);
        }
        pc[jj] = pack2<BF>(v0, v1);
      }
      // Pc buffer i & 1 is free once dV of tile i-2 has been accumulated (long ago, as a rule)
      if (i > 1) {
        if (!mbar_wait(&misc->mma_done[i & 1], ((i >> 1) - 1) & 1, abort_flag, 1605 + g, i)) { ok = false; break; }
      }
      {
        uint8_t* prow = smem + OFF_PC + (i & 1) * PC_BYTES + row * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int chunk = (g * 2 + c) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pc[4 * c], pc[4 * c + 1], pc[4 * c + 2], pc[4 * c + 3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(&misc->e_done);
      if (++st == TST) st = 0;
    }
    ok = ok && mbar_wait(&misc->acc_full, 0, abort_flag, 1611 + g);
    tc_fence_after();
    uint32_t acc[64];
    const size_t grow = size_t(bh) * args.n + size_t(kv_tile) * BKV + row;
    tmem_ld32(tb + T_DV + g * 64, acc);
    tmem_ld32(tb + T_DV + g * 64 + 32, acc + 32);
    tc_wait_ld();
    if (ok && !*abort_flag && kv_tile * BKV + row < args.n) {
      uint4* p = reinterpret_cast<uint4*>(args.dv + grow * DV + g * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 v;
        v.x = pack2<BF>(__uint_as_float(acc[8 * i + 0]), __uint_as_float(acc[8 * i + 1]));
        v.y = pack2<BF>(__uint_as_float(acc[8 * i + 2]), __uint_as_float(acc[8 * i + 3]));
        v.z = pack2<BF>(__uint_as_float(acc[8 * i + 4]), __uint_as_float(acc[8 * i + 5]));
        v.w = pack2<BF>(__uint_as_float(acc[8 * i + 6]), __uint_as_float(acc[8 * i + 7]));
        p[i] = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace da
