// Forward kernel for head dims 32 and 64 (tile sizes, rings and TMEM map: namespace fwd64 in fwd.cuh).
//
// Eight softmax warps: warpgroup b owns branch b, a thread owns a query row and all 64 columns of a score sub-tile.
// The two branches take turns on the exp unit: an mbarrier token (`turn`) lets branch 0 run its pass over sub-tile
// t, then branch 1, then branch 0 over t+1 ...; the token is released after 22 of a pass's 32 element pairs because
// the parked waiter needs ~200 clocks to resume.  Left to themselves both branches reach every phase (wait,
// tcgen05.ld, exp pass, tcgen05.st, arrive) together, since their scores complete together, and the exp unit idles
// during the hand-offs.
// (One 128-column score tile per branch and key tile instead -- no second score buffer; S_b of the next tile issued once
// P_b V of this one has completed, so that the two branches alternate between softmax and MMAs by construction; each
// thread takes its 128 columns in four chunks and holds the 64 packed probabilities until the tile's maximum is known --
// measured 1.08 ms against 0.81 ms at B4 H16 N4096 D64 with 184 registers and 12 bytes spilled: a single warp per
// scheduler runs the exp pass at 28 clocks per element pair, and nothing else fills the exp unit meanwhile.)
#pragma once
#include "fwd.cuh"

namespace da {
namespace fwd64 {
constexpr int MISC_BYTES = 4096;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024; // +1024 for manual alignment
// warps 0-7 softmax (branch = warp >> 2, thread = query row); 8 TMA producer; 9 allocates TMEM and is otherwise idle;
// 10, 11 MMA issuers of branch 1, 2 (S_b and P_b V: S_b of sub-tile t+2 is issued right behind P_b V of sub-tile t, in the
// same thread's issue order -- with a separate S issuer a completion barrier and that warp's wake-up sat between the
// two: 0.804 -> 0.787 ms at B4 H16 N4096 D64): one role warp per scheduler (warp % 4).  Twelve warps, three per scheduler, are launched
// with 168 registers per thread; the role warpgroup then hands registers to the softmax warpgroups (setmaxnreg),
// which hold a whole 64-column sub-tile of scores plus its packed probabilities per thread.  Per scheduler up to
// 2 x 224 + 56 = 3 x 168 are available; measured at B4 H16 N4096 D64, 224 (no spill) and 200 run 5 % slower than 184
// and 168 (about 100 bytes spilled, on the rarely taken rescale path).
constexpr int NUM_THREADS = 384;
#ifndef DA_FWD64_SOFTMAX_REGS
#define DA_FWD64_SOFTMAX_REGS 184
#endif
constexpr int REGS_SOFTMAX = DA_FWD64_SOFTMAX_REGS, REGS_ROLE = 56;
constexpr int WARP_TMA = 8, WARP_S = 9, WARP_PV = 10;
// element pair (of 32) of an exp pass after which the other branch may start its own pass (measured best of 16..28
// at B4 H16 N4096 D64)
constexpr int HANDOVER_AT = 22;
struct Misc {
  uint64_t bar_q;
  uint64_t k_full[KS], k_empty[KS];
  uint64_t v_full[VS], v_empty[VS];
  uint64_t s_full[2][2];     // [branch][buffer]: S sub-tile written by the MMA
  uint64_t p_full[2][2];     // [branch][buffer]: P written by the softmax warpgroup (128 arrivals)
  uint64_t pv_done[2][2];    // [branch][buffer]: P_b V of the sub-tile that used this buffer has completed
  uint64_t o_full;           // everything accumulated
  uint64_t turn[2];
  uint32_t tmem_slot;
  int abort_flag;
  float coef1[BM];     // 1 / l1
  float coef2[BM];     // 1 / l2
  float ssq[2][BM];    // partial sums of squares per column half
};
static_assert(sizeof(Misc) <= MISC_BYTES, "misc area too small");
}  // namespace fwd64


template <bool BF, bool DROP>   // BF: tensors are bf16 instead of fp16; DROP: attention dropout on
__global__ void __launch_bounds__(fwd64::NUM_THREADS, 1)
diffattn_fwd64_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                      const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_y,
                      const __grid_constant__ CUtensorMap tm_a2, const __grid_constant__ CUtensorMap tm_yg,
                      const FwdArgs args) {
  using namespace fwd64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // causal: the later a query tile, the more keys it sees -- the heaviest tiles are launched first so that the grid's tail is light
  const int q_tile = args.causal ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x);
  const int bh = blockIdx.y;
  const int b_idx = bh / args.h;
  const int h_idx = bh % args.h;
  // the last tile may reach past N (TMA fills those rows with zeros); with a causal mask the tiles right of
  // the diagonal tile are skipped altogether
  const int nkv_all = (args.n + BN - 1) / BN;
  const int nkv = (args.causal && q_tile + 1 < nkv_all) ? q_tile + 1 : nkv_all;
  const int nsub = 2 * nkv;          // 64-row sub-tiles

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_q, 1);
        for (int i = 0; i < KS; ++i) { mbar_init(&misc->k_full[i], 1); mbar_init(&misc->k_empty[i], 2); }
    for (int i = 0; i < VS; ++i) { mbar_init(&misc->v_full[i], 1); mbar_init(&misc->v_empty[i], 2); }
    for (int b = 0; b < 2; ++b) {
      for (int u = 0; u < 2; ++u) { mbar_init(&misc->s_full[b][u], 1); mbar_init(&misc->p_full[b][u], 128); }
      for (int u = 0; u < 2; ++u) mbar_init(&misc->pv_done[b][u], 1);
    }
    mbar_init(&misc->o_full, 2);
    mbar_init(&misc->turn[0], 4);
    mbar_init(&misc->turn[1], 4);
    misc->abort_flag = 0;
    mbar_init_fence();
    // The first loads go out before the CTA-wide setup barrier (TMEM allocation, everyone's arrival): the
    // barriers they complete on are initialised above, and the first pass over a ring needs no "empty" wait.
    mbar_expect_tx(&misc->bar_q, 2 * Q_BYTES);
    tma_load_4d(smem + OFF_Q1, &tm_q1, &misc->bar_q, 0, q_tile * BM, h_idx, b_idx);
    tma_load_4d(smem + OFF_Q2, &tm_q2, &misc->bar_q, 0, q_tile * BM, h_idx, b_idx);
    for (int j = 0; j < PRELOAD && j < nkv; ++j) {
      mbar_expect_tx(&misc->k_full[j], 2 * K_BYTES);
      tma_load_4d(smem + OFF_K + j * 2 * K_BYTES, &tm_k1, &misc->k_full[j], 0, j * BN, h_idx, b_idx);
      tma_load_4d(smem + OFF_K + j * 2 * K_BYTES + K_BYTES, &tm_k2, &misc->k_full[j], 0, j * BN, h_idx, b_idx);
      mbar_expect_tx(&misc->v_full[j], V_BYTES);
      tma_load_4d(smem + OFF_V + j * V_BYTES, &tm_v, &misc->v_full[j], 0, j * BN, h_idx, b_idx);
      tma_load_4d(smem + OFF_V + j * V_BYTES + V_BYTES / 2, &tm_v, &misc->v_full[j], 64, j * BN, h_idx, b_idx);
    }
    tma_prefetch_desc(&tm_y); tma_prefetch_desc(&tm_a2);
  }
  if (warp == WARP_S) {
    tmem_alloc(&misc->tmem_slot, 512);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    // ------------------------------- TMA producer -------------------------------
    reg_dec<REGS_ROLE>();
    if (elect_one()) {
      for (int j = PRELOAD; j < nkv; ++j) {
        const int ks = j % KS, vs = j % VS;
        if (!mbar_wait(&misc->k_empty[ks], ((j / KS) & 1) ^ 1, abort_flag, 101, j)) break;
        mbar_expect_tx(&misc->k_full[ks], 2 * K_BYTES);
        tma_load_4d(smem + OFF_K + ks * 2 * K_BYTES, &tm_k1, &misc->k_full[ks], 0, j * BN, h_idx, b_idx);
        tma_load_4d(smem + OFF_K + ks * 2 * K_BYTES + K_BYTES, &tm_k2, &misc->k_full[ks], 0, j * BN, h_idx, b_idx);
        if (!mbar_wait(&misc->v_empty[vs], ((j / VS) & 1) ^ 1, abort_flag, 102, j)) break;
        mbar_expect_tx(&misc->v_full[vs], V_BYTES);
        tma_load_4d(smem + OFF_V + vs * V_BYTES, &tm_v, &misc->v_full[vs], 0, j * BN, h_idx, b_idx);
        tma_load_4d(smem + OFF_V + vs * V_BYTES + V_BYTES / 2, &tm_v, &misc->v_full[vs], 64, j * BN, h_idx, b_idx);
      }
    }
  } else if (warp == WARP_S) {
    // (idle but for the TMEM allocation: completes the role warpgroup, whose registers go to the softmax warpgroups)
    reg_dec<REGS_ROLE>();
  } else if (warp == WARP_PV || warp == WARP_PV + 1) {
    // ------------------- MMA issuer of one branch: S_b(t) = Q_b K_b(sub-tile t)^T, O_b += P_b(t) V(sub-tile t) -------------------
    // One thread, chosen by elect.sync, runs the whole loop.  (A thread picked by comparing the lane id issues
    // tcgen05.mma about three times slower: 152 against 48 clocks per instruction, measured.)
    reg_dec<REGS_ROLE>();
    if (elect_one()) {
      const int br = warp - WARP_PV;
      const uint32_t IDESC_O = make_idesc(BM, 2 * args.d, 0, 1, BF);    // V is MN-major; head dim 32: the 64 real value columns only
      constexpr uint32_t HALF = (SUB * 128) >> 4;
      const uint32_t v_lo0 = sdesc_lo(smem_u32(smem + OFF_V), V_BYTES / 2);
      const uint32_t t_o = tmem_base + T_O + br * 128, t_p = tmem_base + br * 128;
      // This warp issues S_b as well: S_b(t+2) goes into the buffer P_b(t) leaves, right behind P_b(t) V in the same
      // thread's issue order -- no completion barrier and no second warp's wake-up between the two.
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);
      const int kd = args.d >> 4;
      const uint32_t q_lo = sdesc_lo(smem_u32(smem + (br ? OFF_Q2 : OFF_Q1)));
      const uint32_t k_lo0 = sdesc_lo(smem_u32(smem + OFF_K));
      auto issue_s = [&](uint32_t k_lo, int u) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          if (k < kd) mma_ss_lo(t_p + u * SUB, q_lo + k * 2, k_lo + br * (K_BYTES >> 4) + u * HALF + k * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[br][u]);
      };
      int vs = 0, ks = 0;
      uint32_t v_par = 0, k_par = 0;
      bool ok = mbar_wait(&misc->bar_q, 0, abort_flag, 201);
      ok = ok && mbar_wait(&misc->k_full[0], 0, abort_flag, 202);
      if (ok) {
        tc_fence_after();
        issue_s(k_lo0, 0);
        issue_s(k_lo0, 1);
        mma_commit(&misc->k_empty[0]);
        if (++ks == KS) { ks = 0; k_par ^= 1; }
      }
      for (int j = 0; ok && j < nkv; ++j) {
        const uint32_t v_lo = v_lo0 + vs * (V_BYTES >> 4);
        const uint32_t k_lo = k_lo0 + ks * ((2 * K_BYTES) >> 4);       // key tile j+1
        if (!mbar_wait(&misc->v_full[vs], v_par, abort_flag, 205, j)) break;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (!mbar_wait(&misc->p_full[br][u], j & 1, abort_flag, 206 + u, j)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(t_o, t_p + u * SUB + k * 8, v_lo + u * HALF + k * (2048 >> 4), IDESC_O, (j > 0 || u > 0 || k > 0));
          mma_commit(&misc->pv_done[br][u]);
          if (j + 1 < nkv) {
            if (u == 0 && !mbar_wait(&misc->k_full[ks], k_par, abort_flag, 203, j)) { ok = false; break; }
            tc_fence_after();
            issue_s(k_lo, u);
          }
        }
        if (!ok) break;
        if (j + 1 < nkv) {
          mma_commit(&misc->k_empty[ks]);
          if (++ks == KS) { ks = 0; k_par ^= 1; }
        }
        mma_commit(&misc->v_empty[vs]);
        if (++vs == VS) { vs = 0; v_par ^= 1; }
      }
      mma_commit(&misc->o_full);
    }
  } else {
    // ------------------------- softmax warpgroups + epilogue -------------------------
    reg_inc<REGS_SOFTMAX>();
    const int br = warp >> 2;                       // branch handled by this warpgroup
    const int row = (warp & 3) * 32 + lane;         // query row inside the tile = TMEM lane
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t t_s0 = tmem_base + lane_base + br * 128;
    const uint32_t t_o = tmem_base + lane_base + T_O + br * 128;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const f32x2 sl2_2 = pk2(sl2, sl2);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    // dropout: this row's half of every 2x2 block hash, keyed by (seed, batch*head, branch)
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t drow2 = uint32_t(q_tile * BM + row) >> 1;
    const int drow_odd = row & 1;

    for (int t = 0; t < nsub; ++t) {
      const uint32_t t_s = t_s0 + (t & 1) * SUB;
      if (!mbar_wait(&misc->s_full[br][t & 1], (t >> 1) & 1, abort_flag, 301 + br, t)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[SUB];
      tmem_ld32(t_s + 0, sr);
      tmem_ld32(t_s + 32, sr + 32);
      tc_wait_ld();
      {
        // key columns past the sequence end, or right of the diagonal under the causal mask, get a score of
        // -inf (probability 0); nv = number of visible columns of this row in this sub-tile
        int nv = args.n - t * SUB;
        if (args.causal) nv = min(nv, q_tile * BM + row - t * SUB + 1);
        if (nv < SUB) {
#pragma unroll
          for (int i = 0; i < SUB; ++i)
            if (i >= nv) sr[i] = 0xff800000u;
        }
      }
      // One pass: exponentials against the running maximum m_run of the earlier sub-tiles, the row
      // maximum of this sub-tile alongside (independent chains, hidden under the exp unit's latency).
      // If the new maximum exceeds m_run by more than 2^8 (rare; always at t = 0) the pass is redone
      // with the updated maximum after rescaling O_b and l, so P never leaves fp16 range and the final
      // normalisation stays exact.
      float neg = -m_run * sl2;
      f32x2 sum2[2] = {pk2(0.f, 0.f), pk2(0.f, 0.f)};
      float mx[4];
      uint32_t pk[SUB / 2];
#pragma unroll
      for (int c = 0; c < 4; ++c) mx[c] = __uint_as_float(sr[c]);
      if (!mbar_wait(&misc->turn[br], (t + 1 + br) & 1, abort_flag, 321 + br, t)) { ok = false; break; }
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
          // O_b must be quiescent: wait for P_b V of the previous sub-tile, then rescale it
          if (!mbar_wait(&misc->pv_done[br][(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag, 305 + br, t)) { ok = false; break; }
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
      mbar_arrive(&misc->p_full[br][t & 1]);
    }

    // ---- epilogue: every thread runs every barrier; only the global writes depend on `ok`
    ok = ok && mbar_wait(&misc->o_full, 0, abort_flag, 311 + br);
    tc_fence_after();
    const float inv_l = (DROP ? args.drop_scale : 1.f) / l_run;      // kept probabilities are scaled by 1 / (1 - p)
    if (br == 0) misc->coef1[row] = inv_l; else misc->coef2[row] = inv_l;
    named_bar_sync(1, 256);
    const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
    const float c1 = misc->coef1[row];
    const float c2 = misc->coef2[row];
    // this warpgroup owns value columns [64*br, 64*br+64) of both accumulators
    const uint32_t t_o1 = tmem_base + lane_base + T_O + br * 64;
    const uint32_t t_o2 = tmem_base + lane_base + T_O + 128 + br * 64;
    uint32_t o1[64], o2[64];
    tmem_ld32(t_o1, o1);
    tmem_ld32(t_o1 + 32, o1 + 32);
    tmem_ld32(t_o2, o2);
    tmem_ld32(t_o2 + 32, o2 + 32);
    tc_wait_ld();
    float ssq = 0.f;
    const bool pad_half = br * 64 >= 2 * args.d;      // head dim 32: columns 64..127 of the accumulators were never written
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float a2v = pad_half ? 0.f : __uint_as_float(o2[i]) * c2;
      const float av = pad_half ? 0.f : __uint_as_float(o1[i]) * c1 - lam * a2v;
      ssq += av * av;
      o1[i] = __float_as_uint(av);
      o2[i] = __float_as_uint(a2v);
    }
    misc->ssq[br][row] = ssq;
    named_bar_sync(1, 256);
    const int dv_real = 2 * args.d;                      // 128, or 64 when the head dim is 32 (upper columns are padding)
    const float rstd = rsqrtf((misc->ssq[0][row] + misc->ssq[1][row]) / float(dv_real) + args.eps);
    const float yscale = args.rms_norm ? args.out_scale * rstd : 1.f;
    const size_t grow = size_t(bh) * args.n + size_t(q_tile) * BM + row;
    ok = ok && (q_tile * BM + row < args.n);            // rows past the sequence end are computed on zero padding and dropped
    // y and a2 leave through shared memory and the TMA engine: each thread lays its 64 columns into a swizzled
    // [128 rows][64 columns] tile in the (now idle) K ring, and one thread per warpgroup stores the two tiles.
    // (Row-per-thread global stores of 16-byte pieces cost 3.6 us per CTA, 8 % of the kernel at N = 4096.)
    {
      uint8_t* ytile = smem + OFF_K + br * (3 * STORE_TILE_BYTES);
      uint8_t* atile = ytile + STORE_TILE_BYTES;
      uint8_t* gtile = atile + STORE_TILE_BYTES;          // y * gain, only with a gain
      const float4* gp = reinterpret_cast<const float4*>(args.gain + br * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(o1[8 * i + k]) * yscale;
        uint4 av;
        av.x = pack2<BF>(__uint_as_float(o2[8 * i + 0]), __uint_as_float(o2[8 * i + 1]));
        av.y = pack2<BF>(__uint_as_float(o2[8 * i + 2]), __uint_as_float(o2[8 * i + 3]));
        av.z = pack2<BF>(__uint_as_float(o2[8 * i + 4]), __uint_as_float(o2[8 * i + 5]));
        av.w = pack2<BF>(__uint_as_float(o2[8 * i + 6]), __uint_as_float(o2[8 * i + 7]));
        st_swizzled_chunk(ytile, row, i, make_uint4(pack2<BF>(f[0], f[1]), pack2<BF>(f[2], f[3]), pack2<BF>(f[4], f[5]), pack2<BF>(f[6], f[7])));
        st_swizzled_chunk(atile, row, i, av);
        if (args.gain && br * 64 + 8 * i < dv_real) {
          const float4 g0 = __ldg(gp + 2 * i), g1 = __ldg(gp + 2 * i + 1);
          st_swizzled_chunk(gtile, row, i, make_uint4(pack2<BF>(f[0] * g0.x, f[1] * g0.y), pack2<BF>(f[2] * g0.z, f[3] * g0.w),
                                                      pack2<BF>(f[4] * g1.x, f[5] * g1.y), pack2<BF>(f[6] * g1.z, f[7] * g1.w)));
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(2 + br, 128);
      if ((warp & 3) == 0 && elect_one()) {
        if (!*abort_flag && br * 64 < dv_real) {
          tma_store_4d(ytile, &tm_y, br * 64, q_tile * BM, bh, 0);
          tma_store_4d(atile, &tm_a2, br * 64, q_tile * BM, bh, 0);
          if (args.gain) tma_store_4d(gtile, &tm_yg, br * 64, q_tile * BM, bh, 0);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
    }
    if (ok && !*abort_flag) {
      const float lse = m_run * args.sm_scale + logf(l_run);
      if (br == 0) {
        args.lse1[grow] = lse;
        args.rstd[grow] = rstd;
      } else {
        args.lse2[grow] = lse;
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

}  // namespace da
