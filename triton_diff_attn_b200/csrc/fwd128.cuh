// Differential-attention forward for head dim D = 128 (value width 256), sm_100a.
//
// Same roles and TMEM map as the D <= 64 kernel (fwd.cuh, fwd64.cuh): S1/S2 in two 64-column buffers each, O1 and
// O2 128 columns each; eight softmax warps whose two branches take turns on the exp unit; here one warp issues every
// MMA.  Two 256-wide accumulators do not fit in TMEM, so one CTA makes two passes over the key/value sequence, one per
// 128-column half of V: the scores and probabilities are recomputed in the second pass (same values), the row
// statistics are identical in both, and the RMSNorm sum of squares is accumulated over the two passes.  With rms_norm
// the first half of A is parked as 16-bit pairs in registers until the second pass has produced rstd.  Streamed tiles
// are 64 rows: {K1, K2, V half}.
#pragma once
#include "fwd.cuh"
#include "sm100.cuh"

namespace da {

namespace fwd128 {
constexpr int BM = 128, SUB = 64, HD = 128, DV = 256, ST = 3;
constexpr int Q_BYTES = BM * HD * 2;            // 32 KB: two boxes [128 x 64]
constexpr int K_BYTES = SUB * HD * 2;           // 16 KB: two boxes [64 x 64]
constexpr int V_BYTES = SUB * 128 * 2;          // 16 KB: the pass's 128 value columns, two boxes [64 x 64]
constexpr int STAGE_BYTES = 2 * K_BYTES + V_BYTES;   // 48 KB
constexpr int OFF_Q1 = 0, OFF_Q2 = Q_BYTES, OFF_STAGE = 2 * Q_BYTES;   // 64 KB
constexpr int OFF_MISC = OFF_STAGE + ST * STAGE_BYTES;                 // 208 KB
constexpr int MISC_BYTES = 4096;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
// warps 0-7 softmax, 8 TMA, 9 MMA issuer, 10 and 11 idle: they complete the third warpgroup so that it can hand its
// registers to the softmax warpgroups (setmaxnreg works on whole warpgroups): per scheduler up to 2 x 224 + 56 = 3 x 168
// (184, 200 and 224 measured within 2 % of one another at B2 H8 N8192 D128; 168, i.e. no transfer, 2 % slower)
constexpr int NUM_THREADS = 384;
#ifndef DA_FWD128_SOFTMAX_REGS
#define DA_FWD128_SOFTMAX_REGS 184
#endif
constexpr int REGS_SOFTMAX = DA_FWD128_SOFTMAX_REGS, REGS_ROLE = 56;
constexpr int T_O = 256;
constexpr int HANDOVER_AT = 22;   // element pair (of 32) of an exp pass after which the other branch may start (see fwd64.cuh)

struct Misc {
  uint64_t bar_q;
  uint64_t full[ST], empty[ST];
  uint64_t s_full[2][2], p_full[2][2];
  uint64_t o_done[2];
  uint64_t o_full;
  uint64_t turn[2];
  uint32_t tmem_slot;
  int abort_flag;
  float coef1[BM], coef2[BM];
  float ssq[2][BM];
};
static_assert(sizeof(Misc) <= MISC_BYTES, "misc area too small");
}  // namespace fwd128

template <bool BF, bool DROP>
__global__ void __launch_bounds__(fwd128::NUM_THREADS, 1)
diffattn_fwd128_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                       const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                       const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  using namespace fwd128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x, bh = blockIdx.y;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  const int nsub_all = ((args.n + 127) / 128) * 2;     // 64-row sub-tiles, N rounded up to 128 (TMA zero-fills)
  const int nsub = (args.causal && 2 * (q_tile + 1) < nsub_all) ? 2 * (q_tile + 1) : nsub_all;   // causal: stop at the diagonal tile
  const int ntot = 2 * nsub;          // sub-tiles over both passes

  if (warp == 8 && lane == 0) {
    mbar_init(&misc->bar_q, 1);
    for (int i = 0; i < ST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->empty[i], 1); }
    for (int b = 0; b < 2; ++b) {
      for (int u = 0; u < 2; ++u) { mbar_init(&misc->s_full[b][u], 1); mbar_init(&misc->p_full[b][u], 128); }
      mbar_init(&misc->o_done[b], 1);
    }
    mbar_init(&misc->o_full, 1);
    mbar_init(&misc->turn[0], 4);
    mbar_init(&misc->turn[1], 4);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 9) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == 8) {
    reg_dec<REGS_ROLE>();
    if (elect_one()) {
      mbar_expect_tx(&misc->bar_q, 2 * Q_BYTES);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(smem + OFF_Q1 + c * 16384, &tm_q1, &misc->bar_q, c * 64, q_tile * BM, h_idx, b_idx);
        tma_load_4d(smem + OFF_Q2 + c * 16384, &tm_q2, &misc->bar_q, c * 64, q_tile * BM, h_idx, b_idx);
      }
      int st = 0;
      uint32_t par = 1;
      for (int gt = 0; gt < ntot; ++gt) {
        const int pass = gt >= nsub, t = pass ? gt - nsub : gt;
        uint8_t* sp = smem + OFF_STAGE + st * STAGE_BYTES;
        if (!mbar_wait(&misc->empty[st], par, abort_flag, 2101, gt)) break;
        mbar_expect_tx(&misc->full[st], STAGE_BYTES);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(sp + c * 8192, &tm_k1, &misc->full[st], c * 64, t * SUB, h_idx, b_idx);
          tma_load_4d(sp + K_BYTES + c * 8192, &tm_k2, &misc->full[st], c * 64, t * SUB, h_idx, b_idx);
          tma_load_4d(sp + 2 * K_BYTES + c * 8192, &tm_v, &misc->full[st], pass * 128 + c * 64, t * SUB, h_idx, b_idx);
        }
        if (++st == ST) { st = 0; par ^= 1; }
      }
    }
  } else if (warp == 9) {
    reg_dec<REGS_ROLE>();
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);
      constexpr uint32_t IDESC_O = make_idesc(BM, 128, 0, 1, BF);
      const uint32_t q1_lo = sdesc_lo(smem_u32(smem + OFF_Q1)), q2_lo = sdesc_lo(smem_u32(smem + OFF_Q2));
      const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
      const uint32_t tb = tmem_base;
      auto issue_s = [&](uint32_t sp_lo, int u) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ss_lo(tb + u * SUB, q1_lo + (k / 4) * (16384 >> 4) + (k % 4) * 2, sp_lo + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[0][u]);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_ss_lo(tb + 128 + u * SUB, q2_lo + (k / 4) * (16384 >> 4) + (k % 4) * 2,
                    sp_lo + (K_BYTES >> 4) + (k / 4) * (8192 >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[1][u]);
      };
      bool ok = mbar_wait(&misc->bar_q, 0, abort_flag, 2201);
      ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 2202);
      if (ok) {
        tc_fence_after();
        issue_s(st_lo0, 0);
        int st = 0;
        uint32_t par = 0;
        for (int gt = 0; gt < ntot; ++gt) {
          const int u = gt & 1;
          const int t = gt >= nsub ? gt - nsub : gt;
          const uint32_t sp_lo = st_lo0 + st * (STAGE_BYTES >> 4);
          // V half-tile as MN-major B: 128 columns = two atoms 8 KB apart
          const uint32_t v_lo = sp_lo + ((2 * K_BYTES) >> 4) + ((8192u >> 4) << 16) - (1u << 16);
          int st_n = st + 1;
          uint32_t par_n = par;
          if (st_n == ST) { st_n = 0; par_n ^= 1; }
          if (gt + 1 < ntot) {
            if (!mbar_wait(&misc->full[st_n], par_n, abort_flag, 2203, gt)) break;
            tc_fence_after();
            issue_s(st_lo0 + st_n * (STAGE_BYTES >> 4), u ^ 1);
          }
          const uint32_t ph = (gt >> 1) & 1;
          if (!mbar_wait(&misc->p_full[0][u], ph, abort_flag, 2204, gt)) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(tb + T_O, tb + u * SUB + k * 8, v_lo + k * (2048 >> 4), IDESC_O, (t > 0 || k > 0));
          mma_commit(&misc->o_done[0]);
          if (!mbar_wait(&misc->p_full[1][u], ph, abort_flag, 2205, gt)) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(tb + T_O + 128, tb + 128 + u * SUB + k * 8, v_lo + k * (2048 >> 4), IDESC_O, (t > 0 || k > 0));
          mma_commit(&misc->o_done[1]);
          mma_commit(&misc->empty[st]);
          if (t == nsub - 1) mma_commit(&misc->o_full);
          st = st_n;
          par = par_n;
        }
      }
    }
  } else if (warp >= 10) {
    reg_dec<REGS_ROLE>();               // idle warps: only here to complete the warpgroup
  } else {
    reg_inc<REGS_SOFTMAX>();
    const int br = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t t_s0 = tmem_base + lane_base + br * 128;
    const uint32_t t_o = tmem_base + lane_base + T_O + br * 128;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const f32x2 sl2_2 = pk2(sl2, sl2);
    const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
    const size_t grow = size_t(bh) * args.n + size_t(q_tile) * BM + row;
    bool ok = true;
    float ssq_total = 0.f;
    // dropout (same decisions in both passes: they depend on the position only)
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t drow2 = uint32_t(q_tile * BM + row) >> 1;
    const int drow_odd = row & 1;
    uint32_t parked[32];            // first-pass A (this thread's 64 columns) as fp16 pairs, used with rms_norm
#pragma unroll
    for (int i = 0; i < 32; ++i) parked[i] = 0u;

    for (int pass = 0; pass < 2; ++pass) {
      float m_run = -INFINITY, l_run = 0.f;
      for (int t = 0; t < nsub; ++t) {
        const int gt = pass * nsub + t;
        const uint32_t t_s = t_s0 + (gt & 1) * SUB;
        if (!mbar_wait(&misc->s_full[br][gt & 1], (gt >> 1) & 1, abort_flag, 2301 + br, gt)) { ok = false; break; }
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
        float neg = -m_run * sl2;
        f32x2 sum2[2] = {pk2(0.f, 0.f), pk2(0.f, 0.f)};
        float mx[4];
        uint32_t pk[SUB / 2];
#pragma unroll
        for (int c = 0; c < 4; ++c) mx[c] = __uint_as_float(sr[c]);
        if (!mbar_wait(&misc->turn[br], (gt + 1 + br) & 1, abort_flag, 2321 + br, gt)) { ok = false; break; }
        if (t > 0) {
#pragma unroll
          for (int i = 0; i < SUB / 2; ++i) {
            if (i == HANDOVER_AT) { __syncwarp(); if (lane == 0) mbar_arrive(&misc->turn[br ^ 1]); }
            float x0, x1;
            up2(fma2(pk2u(sr[2 * i], sr[2 * i + 1]), sl2_2, pk2(neg, neg)), x0, x1);
            const float p0 = ex2v(x0), p1 = ex2v(x1);
            sum2[i & 1] = add2(sum2[i & 1], pk2(p0, p1));
            pk[i] = pack2<BF>(p0, p1);
            mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < SUB / 2; ++i)
            mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
          __syncwarp(); if (lane == 0) mbar_arrive(&misc->turn[br ^ 1]);
        }
        const float m_new = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        const bool need = (t == 0) || ((m_new - m_run) * sl2 > 8.f);
        if (__any_sync(0xffffffffu, need)) {
          if (t > 0) {
            if (!mbar_wait(&misc->o_done[br], (gt - 1) & 1, abort_flag, 2305 + br, gt)) { ok = false; break; }
            tc_fence_after();
            const float scale = need ? ex2((m_run - m_new) * sl2) : 1.f;
            l_run *= scale;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
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
          l_run += sa + sb;
        }     // the softmax denominator is taken before dropout
        if constexpr (DROP) {
#pragma unroll
          for (int i = 0; i < SUB / 2; ++i)
            pk[i] &= drop_pair_mask(drop_hash(dkey, drow2, uint32_t(t * (SUB / 2) + i)), drow_odd, args.drop_thresh);
        }
        tmem_st32(t_s, pk);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&misc->p_full[br][gt & 1]);
      }

      // ---- epilogue of this pass (value columns [128 pass, 128 pass + 128)); every thread runs every barrier
      ok = ok && mbar_wait(&misc->o_full, pass & 1, abort_flag, 2311 + br, pass);
      tc_fence_after();
      const float inv_l = (DROP ? args.drop_scale : 1.f) / l_run;
      if (br == 0) misc->coef1[row] = inv_l; else misc->coef2[row] = inv_l;
      named_bar_sync(1, 256);
      const float c1 = misc->coef1[row], c2 = misc->coef2[row];
      const uint32_t t_o1 = tmem_base + lane_base + T_O + br * 64;
      const uint32_t t_o2 = tmem_base + lane_base + T_O + 128 + br * 64;
      uint32_t o1[64], o2[64];
      tmem_ld32(t_o1, o1);
      tmem_ld32(t_o1 + 32, o1 + 32);
      tmem_ld32(t_o2, o2);
      tmem_ld32(t_o2 + 32, o2 + 32);
      tc_wait_ld();
      float ssq = 0.f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float a2v = __uint_as_float(o2[i]) * c2;
        const float av = __uint_as_float(o1[i]) * c1 - lam * a2v;
        ssq += av * av;
        o1[i] = __float_as_uint(av);
        o2[i] = __float_as_uint(a2v);
      }
      misc->ssq[br][row] = ssq;
      tc_fence_before();
      named_bar_sync(1, 256);          // all O reads are complete here: the next pass may overwrite O
      ssq_total += misc->ssq[0][row] + misc->ssq[1][row];
      const bool live = ok && !*abort_flag && (q_tile * BM + row < args.n);
      const int col0 = pass * 128 + br * 64;
      if (live) {
        uint4* ap = reinterpret_cast<uint4*>(args.a2 + grow * DV + col0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 av;
          av.x = pack2<BF>(__uint_as_float(o2[8 * i + 0]), __uint_as_float(o2[8 * i + 1]));
          av.y = pack2<BF>(__uint_as_float(o2[8 * i + 2]), __uint_as_float(o2[8 * i + 3]));
          av.z = pack2<BF>(__uint_as_float(o2[8 * i + 4]), __uint_as_float(o2[8 * i + 5]));
          av.w = pack2<BF>(__uint_as_float(o2[8 * i + 6]), __uint_as_float(o2[8 * i + 7]));
          ap[i] = av;
        }
      }
      // eight consecutive output columns of this row: y, and y * gain when a gain is given
      auto put_y = [&](int col, const float (&f)[8]) {
        *reinterpret_cast<uint4*>(args.y + grow * DV + col) =
            make_uint4(pack2<BF>(f[0], f[1]), pack2<BF>(f[2], f[3]), pack2<BF>(f[4], f[5]), pack2<BF>(f[6], f[7]));
        if (args.gain) {
          const float4 g0 = __ldg(reinterpret_cast<const float4*>(args.gain + col));
          const float4 g1 = __ldg(reinterpret_cast<const float4*>(args.gain + col + 4));
          *reinterpret_cast<uint4*>(args.yg + grow * DV + col) =
              make_uint4(pack2<BF>(f[0] * g0.x, f[1] * g0.y), pack2<BF>(f[2] * g0.z, f[3] * g0.w),
                         pack2<BF>(f[4] * g1.x, f[5] * g1.y), pack2<BF>(f[6] * g1.z, f[7] * g1.w));
        }
      };
      if (!args.rms_norm) {
        if (live) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float f[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(o1[8 * i + k]);
            put_y(col0 + 8 * i, f);
          }
        }
      } else if (pass == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) parked[i] = pack2<BF>(__uint_as_float(o1[2 * i]), __uint_as_float(o1[2 * i + 1]));
      } else {
        const float rstd = rsqrtf(ssq_total * (1.f / DV) + args.eps);
        const float ys = args.out_scale * rstd;
        if (live) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float f[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const float2 w = unpack2<BF>(parked[4 * i + c]);
              f[2 * c] = w.x * ys;
              f[2 * c + 1] = w.y * ys;
            }
            put_y(br * 64 + 8 * i, f);
#pragma unroll
            for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(o1[8 * i + k]) * ys;
            put_y(col0 + 8 * i, f);
          }
        }
      }
      if (pass == 1 && live) {
        const float lse = m_run * args.sm_scale + logf(l_run);
        if (br == 0) {
          args.lse1[grow] = lse;
          args.rstd[grow] = rsqrtf(ssq_total * (1.f / DV) + args.eps);
        } else {
          args.lse2[grow] = lse;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace da
