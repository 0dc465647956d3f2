// Differential-attention forward for head dim D = 128 (value width 256), sm_100a.
//
// Two 256-wide accumulators do not fit in TMEM next to the score buffers, so the two branches run in the two CTAs of a
// thread-block cluster (blockIdx.z = branch).  Same softmax scheme as the D <= 64 kernel (fwd.cuh, fwd64.cuh): scores
// in two alternating 64-column TMEM buffers, one exp pass per sub-tile against the stale running maximum, P written
// over its scores as the TMEM A operand of P V.  Streamed tiles are 64 rows: {K_b, V}.  At the end branch 2 hands its
// A2 = O_2 / l_2 in fp32 to branch 1 through distributed shared memory, and branch 1 forms y and rstd.
// (An earlier form kept both branches in one CTA and made two passes over the keys, one per 128-column half of V, with
// the probabilities recomputed in the second: 16 units of B*H*N^2*D and 4 N^2 exponentials per head; it measured
// 1.97 ms against 1.4 ms for this form at B2 H8 N8192 D128.  A form without the cluster -- branch 1 writes A1 as 16-bit
// values into y, a second kernel combines -- was as fast but lost accuracy where A1 - lambda A2 cancels: with bf16
// tensors, lambda 0.8, a causal mask and rms_norm two of 400 seeded cases left the tolerance.  The same
// one-branch-per-CTA form at head dim 64 -- S and O take 256 TMEM columns and 90 KB of shared memory, so two CTAs share
// an SM -- measured 0.84 ms against 0.81 ms for the D <= 64 kernel of fwd64.cuh at B4 H16 N4096 D64: there nothing is
// computed twice to begin with.)
#pragma once
#include "fwd.cuh"
#include "sm100.cuh"

namespace da {

// ------------------------------------------------------------------------------------------------
// One branch per CTA (blockIdx.z; the two CTAs of a query tile are one cluster), one pass: with a single branch the
// whole 256-wide accumulator fits in TMEM next to the score buffers, so nothing is computed twice (12 units of
// B*H*N^2*D and 2 N^2 exponentials per head).
// TMEM: S two 64-column buffers [0,128) | O [128,384).  Warps 0-3 softmax (thread = query row), 4 TMA, 5 MMA issuer.
// ------------------------------------------------------------------------------------------------
namespace fwd128 {
constexpr int BM = 128, SUB = 64, HD = 128, DV = 256, ST = 3;
constexpr int Q_BYTES = BM * HD * 2;            // 32 KB: two boxes [128 x 64]
constexpr int K_BYTES = SUB * HD * 2;           // 16 KB: two boxes [64 x 64]
constexpr int V_BYTES = SUB * DV * 2;           // 32 KB: four boxes [64 x 64]
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;  // 48 KB
constexpr int OFF_Q = 0, OFF_STAGE = Q_BYTES;
constexpr int OFF_MISC = OFF_STAGE + ST * STAGE_BYTES;      // 176 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
// warps 0-3 softmax (thread = query row, all 64 columns of a sub-tile), warp 4 TMA, warp 5 MMA issuer.  (Two softmax
// warps per lane quarter, 32 columns each, exchanging the row maximum through shared memory and a 64-thread named
// barrier once per sub-tile, measured 1.49 ms against 1.38 ms at B2 H8 N8192 D128: the exchange costs more than the
// second warp's help on the exp unit brings.)
constexpr int NUM_THREADS = 192;
constexpr int WARP_TMA = 4, WARP_MMA = 5;
constexpr int T_S = 0, T_O = 128;
struct Misc {
  uint64_t bar_q;
  uint64_t full[ST], empty[ST];
  uint64_t s_full[2], p_full[2];
  uint64_t o_done, o_full;
  uint64_t peer_ready, peer_data;     // arrivals come from the partner CTA of the cluster (the other branch)
  uint32_t tmem_slot;
  int abort_flag;
};
static_assert(sizeof(Misc) <= MISC_BYTES, "misc area too small");
}  // namespace fwd128

template <bool BF, bool DROP>
__global__ void __launch_bounds__(fwd128::NUM_THREADS, 1)
diffattn_fwd128_branch_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                              const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                              const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  using namespace fwd128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the later a query tile, the more keys it sees -- the heaviest tiles are launched first so that the grid's tail is light
  const int q_tile = args.causal ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x), bh = blockIdx.y, br = blockIdx.z;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  const int nsub_all = ((args.n + 127) / 128) * 2;     // 64-row sub-tiles, N rounded up to 128 (TMA zero-fills)
  const int nsub = (args.causal && 2 * (q_tile + 1) < nsub_all) ? 2 * (q_tile + 1) : nsub_all;   // causal: stop at the diagonal tile
  const CUtensorMap* tm_q = br ? &tm_q2 : &tm_q1;
  const CUtensorMap* tm_k = br ? &tm_k2 : &tm_k1;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_q, 1);
    for (int i = 0; i < ST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->empty[i], 1); }
    for (int u = 0; u < 2; ++u) { mbar_init(&misc->s_full[u], 1); mbar_init(&misc->p_full[u], 128); }
    mbar_init(&misc->o_done, 1);
    mbar_init(&misc->o_full, 1);
    mbar_init(&misc->peer_ready, 1);
    mbar_init(&misc->peer_data, 128);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == WARP_MMA) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the partner's mbarriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    if (elect_one()) {
      mbar_expect_tx(&misc->bar_q, Q_BYTES);
      for (int c = 0; c < 2; ++c) tma_load_4d(smem + OFF_Q + c * 16384, tm_q, &misc->bar_q, c * 64, q_tile * BM, h_idx, b_idx);
      int st = 0;
      uint32_t par = 1;
      for (int t = 0; t < nsub; ++t) {
        uint8_t* sp = smem + OFF_STAGE + st * STAGE_BYTES;
        if (!mbar_wait(&misc->empty[st], par, abort_flag, 2101, t)) break;
        mbar_expect_tx(&misc->full[st], STAGE_BYTES);
        for (int c = 0; c < 2; ++c) tma_load_4d(sp + c * 8192, tm_k, &misc->full[st], c * 64, t * SUB, h_idx, b_idx);
        for (int c = 0; c < 4; ++c) tma_load_4d(sp + K_BYTES + c * 8192, &tm_v, &misc->full[st], c * 64, t * SUB, h_idx, b_idx);
        if (++st == ST) { st = 0; par ^= 1; }
      }
    }
  } else if (warp == WARP_MMA) {
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);
      constexpr uint32_t IDESC_O = make_idesc(BM, DV, 0, 1, BF);      // V as MN-major B: four 64-column atoms 8 KB apart
      const uint32_t q_lo = sdesc_lo(smem_u32(smem + OFF_Q));
      const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
      const uint32_t tb = tmem_base;
      auto issue_s = [&](uint32_t sp_lo, int u) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ss_lo(tb + T_S + u * SUB, q_lo + (k / 4) * (16384 >> 4) + (k % 4) * 2, sp_lo + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[u]);
      };
      bool ok = mbar_wait(&misc->bar_q, 0, abort_flag, 2201);
      ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 2202);
      if (ok) {
        tc_fence_after();
        issue_s(st_lo0, 0);
        int st = 0;
        uint32_t par = 0;
        for (int t = 0; t < nsub; ++t) {
          const int u = t & 1;
          const uint32_t sp_lo = st_lo0 + st * (STAGE_BYTES >> 4);
          const uint32_t v_lo = sp_lo + (K_BYTES >> 4) + ((8192u >> 4) << 16) - (1u << 16);
          int st_n = st + 1;
          uint32_t par_n = par;
          if (st_n == ST) { st_n = 0; par_n ^= 1; }
          if (t + 1 < nsub) {
            if (!mbar_wait(&misc->full[st_n], par_n, abort_flag, 2203, t)) break;
            tc_fence_after();
            issue_s(st_lo0 + st_n * (STAGE_BYTES >> 4), u ^ 1);
          }
          if (!mbar_wait(&misc->p_full[u], (t >> 1) & 1, abort_flag, 2204, t)) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(tb + T_O, tb + T_S + u * SUB + k * 8, v_lo + k * (2048 >> 4), IDESC_O, (t > 0 || k > 0));
          mma_commit(&misc->o_done);
          mma_commit(&misc->empty[st]);
          if (t == nsub - 1) mma_commit(&misc->o_full);
          st = st_n;
          par = par_n;
        }
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const uint32_t lane_base = uint32_t(warp * 32) << 16;
    const uint32_t t_s0 = tmem_base + lane_base + T_S;
    const uint32_t t_o = tmem_base + lane_base + T_O;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const f32x2 sl2_2 = pk2(sl2, sl2);
    const size_t grow = size_t(bh) * args.n + size_t(q_tile) * BM + row;
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t drow2 = uint32_t(q_tile * BM + row) >> 1;
    const int drow_odd = row & 1;
    bool ok = true;
    float m_run = -INFINITY, l_run = 0.f;
    for (int t = 0; t < nsub; ++t) {
      const uint32_t t_s = t_s0 + (t & 1) * SUB;
      if (!mbar_wait(&misc->s_full[t & 1], (t >> 1) & 1, abort_flag, 2301 + br, t)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[SUB];
      tmem_ld32(t_s + 0, sr);
      tmem_ld32(t_s + 32, sr + 32);
      tc_wait_ld();
      {
        int nv = args.n - t * SUB;             // visible key columns of this row in this sub-tile; the rest get -inf
        if (args.causal) nv = min(nv, q_tile * BM + row - t * SUB + 1);
        if (nv < SUB) {
#pragma unroll
          for (int i = 0; i < SUB; ++i)
            if (i >= nv) sr[i] = 0xff800000u;
        }
      }
      // one pass against the stale running maximum, the sub-tile's own maximum alongside (see fwd64.cuh)
      float neg = -m_run * sl2;
      f32x2 sum2[2] = {pk2(0.f, 0.f), pk2(0.f, 0.f)};
      float mx[4];
      uint32_t pk[SUB / 2];
#pragma unroll
      for (int c = 0; c < 4; ++c) mx[c] = __uint_as_float(sr[c]);
      if (t > 0) {
#pragma unroll
        for (int i = 0; i < SUB / 2; ++i) {
          float x0, x1;
          up2(fma2(pk2u(sr[2 * i], sr[2 * i + 1]), sl2_2, pk2(neg, neg)), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          sum2[i & 1] = add2(sum2[i & 1], pk2(p0, p1));
          pk[i] = pack2<BF>(p0, p1);
          mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < SUB / 2; ++i)
          mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
      }
      const float m_new = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const bool need = (t == 0) || ((m_new - m_run) * sl2 > 8.f);
      if (__any_sync(0xffffffffu, need)) {
        if (t > 0) {
          // O must be quiescent: wait for P V of the previous sub-tile, then rescale it
          if (!mbar_wait(&misc->o_done, (t - 1) & 1, abort_flag, 2305 + br, t)) { ok = false; break; }
          tc_fence_after();
          const float scale = need ? ex2((m_run - m_new) * sl2) : 1.f;
          l_run *= scale;
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * scale);
            tmem_st32(t_o + c * 32, o);
          }
        }
        if (need) m_run = m_new;
        neg = -m_run * sl2;
        sum2[0] = sum2[1] = pk2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < SUB / 2; ++i) {
          float x0, x1;
          up2(fma2(pk2u(sr[2 * i], sr[2 * i + 1]), sl2_2, pk2(neg, neg)), x0, x1);
          const float p0 = ex2(x0), p1 = ex2(x1);
          sum2[i & 1] = add2(sum2[i & 1], pk2(p0, p1));
          pk[i] = pack2<BF>(p0, p1);
        }
      }
      {
        float sa, sb;
        up2(add2(sum2[0], sum2[1]), sa, sb);
        l_run += sa + sb;                       // the softmax denominator is taken before dropout
      }
      if constexpr (DROP) {
#pragma unroll
        for (int i = 0; i < SUB / 2; ++i)
          pk[i] &= drop_pair_mask(drop_hash(dkey, drow2, uint32_t(t * (SUB / 2) + i)), drow_odd, args.drop_thresh);
      }
      tmem_st32(t_s, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->p_full[t & 1]);
    }

    // ---- epilogue.  The two CTAs of a cluster hold A1 = O_1 / l_1 (branch 1) and A2 = O_2 / l_2 (branch 2) of the same 128
    // query rows.  Branch 2 writes a2 and hands its A2 in fp32 to branch 1 through distributed shared memory (into branch
    // 1's key/value ring, idle by then); branch 1 forms y = RMSNorm(A1 - lambda A2) (1 - lambda_init) and rstd.
    // Every thread runs every barrier; only the global writes depend on `ok`.
    ok = mbar_wait(&misc->o_full, 0, abort_flag, 2311 + br) && ok;
    tc_fence_after();
    const float inv_l = (DROP ? args.drop_scale : 1.f) / l_run;
    const bool live = ok && !*abort_flag && (q_tile * BM + row < args.n);
    // exchange tile: 64 chunks of four floats per row, chunk-major (chunk c of row r at (c * 128 + r) * 16 bytes), so that
    // the 32 rows of a warp touch consecutive 16-byte words
    uint8_t* xtile = smem + OFF_STAGE;
    if (br == 1) {
      const uint32_t x_remote = cluster_map(smem_u32(xtile), 0);
      ok = mbar_wait_cluster(&misc->peer_ready, 0, abort_flag, 2313) && ok;       // branch 1's ring is idle
      __half* dst = args.a2 + grow * DV;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + c * 32, o);
        tc_wait_ld();
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(o[i]) * inv_l;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          cluster_st_v4(x_remote + uint32_t(((c * 8 + i) * BM + row) * 16), f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        if (live) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * i) =
                make_uint4(pack2<BF>(f[8 * i + 0], f[8 * i + 1]), pack2<BF>(f[8 * i + 2], f[8 * i + 3]),
                           pack2<BF>(f[8 * i + 4], f[8 * i + 5]), pack2<BF>(f[8 * i + 6], f[8 * i + 7]));
        }
      }
      cluster_mbar_arrive(cluster_map(smem_u32(&misc->peer_data), 0));
      if (live) args.lse2[grow] = m_run * args.sm_scale + logf(l_run);
    } else {
      if (threadIdx.x == 0) cluster_mbar_arrive(cluster_map(smem_u32(&misc->peer_ready), 1));
      const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
      ok = mbar_wait_cluster(&misc->peer_data, 0, abort_flag, 2314) && ok;
      const bool live0 = live && ok && !*abort_flag;
      const float4* xrow = reinterpret_cast<const float4*>(xtile) + row;
      // first pass: sum of squares of A = A1 - lambda A2 (the accumulator and the exchange tile are read again below);
      // without rms_norm only rstd needs it, and it is gathered in the second pass
      float ssq = 0.f;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        if (!args.rms_norm) break;
        uint32_t o[32];
        tmem_ld32(t_o + c * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 z = xrow[(c * 8 + i) * BM];
          const float a0 = __uint_as_float(o[4 * i + 0]) * inv_l - lam * z.x, a1 = __uint_as_float(o[4 * i + 1]) * inv_l - lam * z.y;
          const float a2 = __uint_as_float(o[4 * i + 2]) * inv_l - lam * z.z, a3 = __uint_as_float(o[4 * i + 3]) * inv_l - lam * z.w;
          ssq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
      }
      const float ys = args.rms_norm ? args.out_scale * rsqrtf(ssq * (1.f / DV) + args.eps) : 1.f;
      float ssq2 = 0.f;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + c * 32, o);
        tc_wait_ld();
        float f[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 z = xrow[(c * 8 + i) * BM];
          const float a0 = __uint_as_float(o[4 * i + 0]) * inv_l - lam * z.x, a1 = __uint_as_float(o[4 * i + 1]) * inv_l - lam * z.y;
          const float a2 = __uint_as_float(o[4 * i + 2]) * inv_l - lam * z.z, a3 = __uint_as_float(o[4 * i + 3]) * inv_l - lam * z.w;
          ssq2 += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
          f[4 * i + 0] = a0 * ys; f[4 * i + 1] = a1 * ys; f[4 * i + 2] = a2 * ys; f[4 * i + 3] = a3 * ys;
        }
        if (live0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c * 32 + 8 * i;
            *reinterpret_cast<uint4*>(args.y + grow * DV + col) =
                make_uint4(pack2<BF>(f[8 * i + 0], f[8 * i + 1]), pack2<BF>(f[8 * i + 2], f[8 * i + 3]),
                           pack2<BF>(f[8 * i + 4], f[8 * i + 5]), pack2<BF>(f[8 * i + 6], f[8 * i + 7]));
            if (args.gain) {
              const float4 g0 = __ldg(reinterpret_cast<const float4*>(args.gain + col));
              const float4 g1 = __ldg(reinterpret_cast<const float4*>(args.gain + col + 4));
              *reinterpret_cast<uint4*>(args.yg + grow * DV + col) =
                  make_uint4(pack2<BF>(f[8 * i + 0] * g0.x, f[8 * i + 1] * g0.y), pack2<BF>(f[8 * i + 2] * g0.z, f[8 * i + 3] * g0.w),
                             pack2<BF>(f[8 * i + 4] * g1.x, f[8 * i + 5] * g1.y), pack2<BF>(f[8 * i + 6] * g1.z, f[8 * i + 7] * g1.w));
            }
          }
        }
      }
      if (live0) {
        args.lse1[grow] = m_run * args.sm_scale + logf(l_run);
        args.rstd[grow] = rsqrtf(ssq2 * (1.f / DV) + args.eps);
      }
    }
  }

  // neither CTA leaves while its partner may still arrive on its barriers or write into its shared memory
  cluster_sync_all();
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace da
