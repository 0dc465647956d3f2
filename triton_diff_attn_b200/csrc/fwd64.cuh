// Forward kernel for head dims 32 and 64 (tile sizes, rings and TMEM map: namespace fwd64 in fwd.cuh).
//
// Sixteen softmax warps, four per scheduler: each row of a 64-column score sub-tile is split between two threads
// (32 columns each, warps `half` 0 and 1 of a branch), which exchange the row maximum once per sub-tile through
// shared memory and a 64-thread named barrier so that both scale by the same maximum.  The two branches take
// turns on the exp unit (mbarrier `turn`), handing it over before a pass ends.  History of this choice, at config
// 2: eight softmax warps owning full 64-column rows, 1.06 ms (one pass ~1250 clocks against 1024 of exp-unit
// work, every wait / tcgen05.ld / st / arrive exposed); sixteen warps without turns, 1.06 ms (all four warps of
// a scheduler reach every phase together, so the exp unit idles during the hand-offs all the same); with turns
// 0.985 ms.
#pragma once
#include "fwd.cuh"

namespace da {

namespace fwd64 {
constexpr int NUM_THREADS = 640;   // 16 softmax warps + 4 role warps, five per scheduler, <= 102 registers each
constexpr int WARP_TMA = 16, WARP_S = 17, WARP_PV = 18;    // one role warp per scheduler (warp % 4)
constexpr int MISC_BYTES = 12288;
// pair index (of 16) of an exp pass after which the other branch may start its own pass; measured at c2:
// 3 -> 1.05 ms, 7 -> 1.00, 9 and 11 -> 0.985, 13 -> 1.00, 15 (the end of the pass) -> 1.09 (no alternation: 1.06).
// Turns of two sub-tiles per branch instead of one: 1.23 ms (a branch's own hand-offs are no longer covered).
constexpr int HANDOVER_AT = 11;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
// named barriers: 1..8 the two warps of a (branch, row quarter); 9 all softmax threads; 10, 11 the 256 threads
// that fill one 64-column store tile
struct Misc {
  uint64_t bar_q;
  uint64_t k_full[KS], k_empty[KS];
  uint64_t v_full[VS], v_empty[VS];
  uint64_t s_full[2][2];     // [branch][buffer]: S sub-tile written by the MMA
  uint64_t p_full[2][2];     // [branch][buffer]: P written by both halves (256 arrivals)
  uint64_t pv_done[2][2];    // [branch][buffer]: P_b V of the sub-tile that used this buffer has completed
  uint64_t o_full;
  uint32_t tmem_slot;
  int abort_flag;
  uint64_t turn[2];          // [branch]: that branch may run its next exp pass (8 arrivals: one per warp of the other branch)
  float xmax[2][2][2][BM];   // [sub-tile parity][branch][half][row]: row maximum of a thread's 32 columns
  float lpart[2][2][BM];     // [branch][half][row]: that thread's share of the softmax denominator
  float ssq[4][BM];          // partial sums of squares per 32-column group
};
static_assert(sizeof(Misc) <= MISC_BYTES, "misc area too small");
}  // namespace fwd64

// O_b[:, 64 columns from t_o] *= scale for this thread's row.  Rare (the running maximum grew by more than 2^8):
// kept out of line so that its 32 transfer registers do not weigh on the exp loop's register budget.
__device__ __noinline__ void fwd64_rescale_o(uint32_t t_o, float scale) {
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t o[32];
    tmem_ld32(t_o + c * 32, o);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * scale);
    tmem_st32(t_o + c * 32, o);
  }
}

template <bool BF, bool DROP>
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
  const int q_tile = blockIdx.x;
  const int bh = blockIdx.y;
  const int b_idx = bh / args.h;
  const int h_idx = bh % args.h;
  const int nkv_all = (args.n + BN - 1) / BN;
  const int nkv = (args.causal && q_tile + 1 < nkv_all) ? q_tile + 1 : nkv_all;   // causal: stop at the diagonal tile
  const int nsub = 2 * nkv;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_q, 1);
    for (int i = 0; i < KS; ++i) { mbar_init(&misc->k_full[i], 1); mbar_init(&misc->k_empty[i], 1); }
    for (int i = 0; i < VS; ++i) { mbar_init(&misc->v_full[i], 1); mbar_init(&misc->v_empty[i], 2); }
    for (int b = 0; b < 2; ++b)
      for (int u = 0; u < 2; ++u) {
        mbar_init(&misc->s_full[b][u], 1);
        mbar_init(&misc->p_full[b][u], 256);
        mbar_init(&misc->pv_done[b][u], 1);
      }
    mbar_init(&misc->o_full, 2);
    mbar_init(&misc->turn[0], 8);
    mbar_init(&misc->turn[1], 8);
    misc->abort_flag = 0;
    mbar_init_fence();
    // first loads before the CTA-wide setup barrier (their barriers exist; a first ring pass needs no "empty" wait)
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
  if (warp == WARP_S) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    // ------------------------------- TMA producer -------------------------------
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
    // ------------------- S issuer: S_b(t) = Q_b K_b(sub-tile t)^T for both branches -------------------
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);
      constexpr uint32_t HALF = (SUB * 128) >> 4;
      const uint32_t q1_lo = sdesc_lo(smem_u32(smem + OFF_Q1)), q2_lo = sdesc_lo(smem_u32(smem + OFF_Q2));
      const uint32_t k_lo0 = sdesc_lo(smem_u32(smem + OFF_K));
      bool ok = mbar_wait(&misc->bar_q, 0, abort_flag, 201);
      int ks = 0;
      uint32_t k_par = 0;
      for (int j = 0; ok && j < nkv; ++j) {
        const uint32_t k_lo = k_lo0 + ks * ((2 * K_BYTES) >> 4);
        if (!mbar_wait(&misc->k_full[ks], k_par, abort_flag, 202, j)) break;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int br = 0; br < 2; ++br) {
#ifdef DA_TIMING
            const bool tm_on = (blockIdx.x == 3 && blockIdx.y == 1) && j >= 8 && j < 12;
            const int tm_base = 2048 + (((j - 8) * 2 + u) * 2 + br) * 4;
#endif
            DA_TS(0);
            if (j > 0) {
              if (!mbar_wait(&misc->pv_done[br][u], (j - 1) & 1, abort_flag, 203 + u, j)) { ok = false; break; }
            }
            tc_fence_after();
            DA_TS(1);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k)
              mma_ss_lo(tmem_base + br * 128 + u * SUB, (br ? q2_lo : q1_lo) + k * 2,
                        k_lo + br * (K_BYTES >> 4) + u * HALF + k * 2, IDESC_S, k > 0);
            mma_commit(&misc->s_full[br][u]);
            DA_TS(2);
          }
          if (!ok) break;
        }
        mma_commit(&misc->k_empty[ks]);
        if (++ks == KS) { ks = 0; k_par ^= 1; }
      }
    }
  } else if (warp == WARP_PV || warp == WARP_PV + 1) {
    // ------------------- P V issuer of one branch: O_b += P_b(t) V(sub-tile t) -------------------
    if (elect_one()) {
      const int br = warp - WARP_PV;
      constexpr uint32_t IDESC_O = make_idesc(BM, DV, 0, 1, BF);
      constexpr uint32_t HALF = (SUB * 128) >> 4;
      const uint32_t v_lo0 = sdesc_lo(smem_u32(smem + OFF_V), V_BYTES / 2);
      const uint32_t t_o = tmem_base + T_O + br * 128, t_p = tmem_base + br * 128;
      int vs = 0;
      uint32_t v_par = 0;
      bool ok = true;
      for (int j = 0; ok && j < nkv; ++j) {
        const uint32_t v_lo = v_lo0 + vs * (V_BYTES >> 4);
        if (!mbar_wait(&misc->v_full[vs], v_par, abort_flag, 205, j)) break;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#ifdef DA_TIMING
          const bool tm_on = (blockIdx.x == 3 && blockIdx.y == 1) && j >= 8 && j < 12;
          const int tm_base = 2304 + (((j - 8) * 2 + u) * 2 + br) * 4;
#endif
          DA_TS(0);
          if (!mbar_wait(&misc->p_full[br][u], j & 1, abort_flag, 206 + u, j)) { ok = false; break; }
          tc_fence_after();
          DA_TS(1);
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            mma_ts_lo(t_o, t_p + u * SUB + k * 8, v_lo + u * HALF + k * (2048 >> 4), IDESC_O, (j > 0 || u > 0 || k > 0));
          mma_commit(&misc->pv_done[br][u]);
          DA_TS(2);
        }
        mma_commit(&misc->v_empty[vs]);
        if (++vs == VS) { vs = 0; v_par ^= 1; }
      }
      mma_commit(&misc->o_full);
    }
  } else {
    // ------------------------- softmax warps + epilogue -------------------------
    const int br = warp >> 3;                        // branch
    const int half = (warp >> 2) & 1;                // which 32 of a sub-tile's 64 columns
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;             // query row inside the tile = TMEM lane
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t t_s0 = tmem_base + lane_base + br * 128;
    const uint32_t t_o = tmem_base + lane_base + T_O + br * 128 + half * 64;   // the 64 columns of O_b this thread rescales
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const int pair_bar = 1 + br * 4 + quarter;       // the two warps that share these 32 rows of this branch
    float m_run = -INFINITY, l_run = 0.f;            // running maximum (same in both halves), own share of the denominator
    bool ok = true;
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t drow2 = uint32_t(q_tile * BM + row) >> 1;
    const int drow_odd = row & 1;

    int synced = 0;                                  // pair barriers passed so far
    for (int t = 0; t < nsub; ++t) {
      const int u = t & 1;
      const uint32_t t_s = t_s0 + u * SUB;
#ifdef DA_TIMING
      const bool tm_on = (blockIdx.x == 3 && blockIdx.y == 1 && lane == 0) && t >= 16 && t < 24;
      const int tm_base = warp * 64 + (t - 16) * 8;
#endif
      DA_TS(0);
      if (!mbar_wait(&misc->s_full[br][u], (t >> 1) & 1, abort_flag, 301 + br, t)) { ok = false; break; }
      tc_fence_after();
      DA_TS(1);
      uint32_t sr[32];
      tmem_ld32(t_s + half * 32, sr);
      tc_wait_ld();
      DA_TS(2);
      {
        // key columns past the sequence end, or right of the diagonal under the causal mask: score -inf
        const int c_first = t * SUB + half * 32;
        int nv = args.n - c_first;
        if (args.causal) nv = min(nv, q_tile * BM + row - c_first + 1);
        if (nv < 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= nv) sr[i] = 0xff800000u;
        }
      }
      // One pass against the running maximum of the earlier sub-tiles, the maximum of these 32 columns alongside;
      // redone with the new maximum (after rescaling O_b and l) only if that exceeds m_run by more than 2^8.
      float neg = -m_run * sl2;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      float mx[4];
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) mx[c] = __uint_as_float(sr[c]);
      // The two branches take turns on the exp unit: branch 0 runs pass t, then branch 1 runs pass t, then branch 0
      // pass t+1 ...  Left to themselves all four warps of a scheduler reach their passes together (both branches'
      // scores become ready together) and then wait, load, store and hand over together, with the exp unit idle;
      // alternating, one branch's hand-over runs under the other's exponentials.
      if (!mbar_wait(&misc->turn[br], (t + 1 + br) & 1, abort_flag, 321 + br, t)) { ok = false; break; }
      DA_TS(7);
      if (t > 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2v(fmaf(__uint_as_float(sr[2 * i]), sl2, neg));
          const float p1 = ex2v(fmaf(__uint_as_float(sr[2 * i + 1]), sl2, neg));
          sum[(2 * i) & 3] += p0;
          sum[(2 * i + 1) & 3] += p1;
          pk[i] = pack2<BF>(p0, p1);
          mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
          if (i == HANDOVER_AT) {
            // hand the exp unit over before this pass ends: the other branch needs ~200 clocks to wake up
            __syncwarp();
            if (lane == 0) mbar_arrive(&misc->turn[br ^ 1]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
        __syncwarp();
        if (lane == 0) mbar_arrive(&misc->turn[br ^ 1]);
      }
      // the row's maximum over all 64 columns: exchange with the thread that holds the other 32 (slots alternate
      // with the sub-tile parity, so a slot is rewritten only after its reader has passed the next barrier)
      const float m_loc = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      DA_TS(3);
      misc->xmax[u][br][half][row] = m_loc;
      named_bar_sync(pair_bar, 64);
      ++synced;
      DA_TS(4);
      const float m_new = fmaxf(m_loc, misc->xmax[u][br][half ^ 1][row]);
      const bool need = (t == 0) || ((m_new - m_run) * sl2 > 8.f);
      if (__any_sync(0xffffffffu, need)) {          // same outcome in both warps of the pair: they hold the same rows
        if (t > 0) {
          if (!mbar_wait(&misc->pv_done[br][(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag, 305 + br, t)) { ok = false; break; }
          tc_fence_after();
          const float scale = need ? ex2((m_run - m_new) * sl2) : 1.f;
          l_run *= scale;
          fwd64_rescale_o(t_o, scale);
        }
        if (need) m_run = m_new;
        neg = -m_run * sl2;
#pragma unroll
        for (int c = 0; c < 4; ++c) sum[c] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2(fmaf(__uint_as_float(sr[2 * i]), sl2, neg));
          const float p1 = ex2(fmaf(__uint_as_float(sr[2 * i + 1]), sl2, neg));
          sum[(2 * i) & 3] += p0;
          sum[(2 * i + 1) & 3] += p1;
          pk[i] = pack2<BF>(p0, p1);
        }
      }
      l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);     // the softmax denominator is taken before dropout
      if constexpr (DROP) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pk[i] &= drop_pair_mask(drop_hash(dkey, drow2, uint32_t(t * (SUB / 2) + half * 16 + i)), drow_odd, args.drop_thresh);
      }
      // P (16-bit, two per column) over the first 32 columns of the score buffer: this half's 32 values in 16 of them.
      // Both threads of the row have their scores in registers since the barrier above, so the overlap is safe.
      DA_TS(5);
      tmem_st16(t_s + half * 16, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->p_full[br][u]);
      DA_TS(6);
    }

    // A warp that left the loop early (a bounded wait expired) arrives, without blocking, on the pair barriers it
    // skipped: its partner may have got past the same wait a moment earlier and would otherwise sit in bar.sync.
    for (; synced < nsub; ++synced) named_bar_arrive(pair_bar, 64);

    // ---- epilogue: every thread runs every barrier; only the global writes depend on `ok`
    ok = ok && mbar_wait(&misc->o_full, 0, abort_flag, 311 + br);
    tc_fence_after();
    misc->lpart[br][half][row] = l_run;
    named_bar_sync(9, 512);
    const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
    const float dsc = DROP ? args.drop_scale : 1.f;       // kept probabilities are scaled by 1 / (1 - p)
    const float l1 = misc->lpart[0][0][row] + misc->lpart[0][1][row];
    const float l2 = misc->lpart[1][0][row] + misc->lpart[1][1][row];
    const float c1 = dsc / l1, c2 = dsc / l2;
    const int w4 = br * 2 + half;                         // owns value columns [32 w4, 32 w4 + 32) of both accumulators
    uint32_t o1[32], o2[32];
    tmem_ld32(tmem_base + lane_base + T_O + w4 * 32, o1);
    tmem_ld32(tmem_base + lane_base + T_O + 128 + w4 * 32, o2);
    tc_wait_ld();
    float ssq = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float a2v = __uint_as_float(o2[i]) * c2;
      const float av = __uint_as_float(o1[i]) * c1 - lam * a2v;
      ssq += av * av;
      o1[i] = __float_as_uint(av);
      o2[i] = __float_as_uint(a2v);
    }
    misc->ssq[w4][row] = ssq;
    named_bar_sync(9, 512);
    const int dv_real = 2 * args.d;                       // 128, or 64 when the head dim is 32 (upper columns are padding)
    const float rstd = rsqrtf(((misc->ssq[0][row] + misc->ssq[1][row]) + (misc->ssq[2][row] + misc->ssq[3][row])) / float(dv_real) + args.eps);
    const float yscale = args.rms_norm ? args.out_scale * rstd : 1.f;
    {
      // y, a2 (and y * gain) leave through swizzled [128][64] tiles in the idle K ring and the TMA engine; the two
      // warpgroups of a branch index fill one tile of each (32 columns = four 16-byte chunks per thread)
      const int tg = w4 >> 1;
      uint8_t* ytile = smem + OFF_K + tg * (3 * STORE_TILE_BYTES);
      uint8_t* atile = ytile + STORE_TILE_BYTES;
      uint8_t* gtile = atile + STORE_TILE_BYTES;
      const float4* gp = reinterpret_cast<const float4*>(args.gain + w4 * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(o1[8 * i + k]) * yscale;
        uint4 av;
        av.x = pack2<BF>(__uint_as_float(o2[8 * i + 0]), __uint_as_float(o2[8 * i + 1]));
        av.y = pack2<BF>(__uint_as_float(o2[8 * i + 2]), __uint_as_float(o2[8 * i + 3]));
        av.z = pack2<BF>(__uint_as_float(o2[8 * i + 4]), __uint_as_float(o2[8 * i + 5]));
        av.w = pack2<BF>(__uint_as_float(o2[8 * i + 6]), __uint_as_float(o2[8 * i + 7]));
        const int chunk = (w4 & 1) * 4 + i;
        st_swizzled_chunk(ytile, row, chunk, make_uint4(pack2<BF>(f[0], f[1]), pack2<BF>(f[2], f[3]), pack2<BF>(f[4], f[5]), pack2<BF>(f[6], f[7])));
        st_swizzled_chunk(atile, row, chunk, av);
        if (args.gain && w4 * 32 + 8 * i < dv_real) {
          const float4 g0 = __ldg(gp + 2 * i), g1 = __ldg(gp + 2 * i + 1);
          st_swizzled_chunk(gtile, row, chunk, make_uint4(pack2<BF>(f[0] * g0.x, f[1] * g0.y), pack2<BF>(f[2] * g0.z, f[3] * g0.w),
                                                          pack2<BF>(f[4] * g1.x, f[5] * g1.y), pack2<BF>(f[6] * g1.z, f[7] * g1.w)));
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(10 + tg, 256);
      if ((warp & 7) == 0 && elect_one()) {
        if (!*abort_flag && tg * 64 < dv_real) {
          tma_store_4d(ytile, &tm_y, tg * 64, q_tile * BM, bh, 0);
          tma_store_4d(atile, &tm_a2, tg * 64, q_tile * BM, bh, 0);
          if (args.gain) tma_store_4d(gtile, &tm_yg, tg * 64, q_tile * BM, bh, 0);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
    }
    if (ok && !*abort_flag && half == 0 && q_tile * BM + row < args.n) {
      const size_t grow = size_t(bh) * args.n + size_t(q_tile) * BM + row;
      const float lse = m_run * args.sm_scale + logf(br ? l2 : l1);
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
