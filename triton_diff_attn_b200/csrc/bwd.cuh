// Differential-attention backward for sm_100a, head dim D = 64 (value width 128).
//
// Three kernels (the default form of the backward) replace the reference's single Triton backward
// (src/kernel.py:221-458); bwd_fused64.cuh holds the optional form that merges 2 and 3:
//   1. bwd_pre      per row: dA = RMSNorm-backward(dY) (src/kernel.py:283-290), E1, E2 row sums
//                   (the reference's D1 and D2/(-lambda), :295-296), d(lambda) = -sum E2 with one
//                   atomic per CTA (division-free; the reference divides by lambda+eps, :293).
//   2. bwd_dkdv64   key/value-stationary: S^T, dP^T on tensor cores, dV += (P1-lam P2)^T dA,
//                   dK_b += dS_b^T Q_b (src/kernel.py:410-424).
//   3. bwd_dq64     query-stationary: dQ_b += dS_b K_b (src/kernel.py:426-436); every dQ tile has one
//                   owner CTA, so the accumulation is race-free and deterministic.
// Both tensor-core kernels recompute P_b = exp(s S_b - lse_b) from the saved logsumexp.
#pragma once
#include "sm100.cuh"
#include "fwd.cuh"

namespace da {

struct BwdArgs {
  const __half* y;      // [B*H, N, 2D]
  const __half* a2;     // [B*H, N, 2D]
  const __half* dy;     // [B*H, N, 2D] dense
  const float* lse1;
  const float* lse2;
  const float* rstd;
  __half* da;           // workspace [B*H, N, 2D]
  float4* stats;        // workspace, 16 bytes per row of [B*H, n_pad], NEGATED and interleaved by row pairs (see stat_row):
                        // x = -lse1*log2e, y = -(lse2*log2e - log2|lam|), z = -E1, w = -sg*E2 with sg = -sign(lam)
  __half* dq1; __half* dq2; __half* dk1; __half* dk2; __half* dv;   // dense
  float* dlambda;
  const void* lambda_ptr;
  int lambda_dtype;
  float sm_scale;
  float out_scale;      // 1 - lambda_init
  int rms_norm;
  int n;
  int h;
  int d;                // real head dim (64, or 32 with zero-filled padding in the 64-wide tiles)
  int causal;           // 1: query row i sees key columns j <= i only
  int n_pad;            // N rounded up to 128: row pitch of `stats` per (batch, head); rows N..n_pad-1 hold
                        // x = y = -inf, z = w = 0, which makes the probabilities of out-of-range query rows exactly 0
  long long rows;       // B*H*N
  uint32_t drop_thresh; // dropout: 0 = off (see sm100.cuh); must equal the forward's
  uint32_t seed_lo, seed_hi;
  float drop_scale;     // 256 / (256 - drop_thresh)
  const float* gain;    // NULL, or fp32 [2D]: then dy is the gradient of y * gain, and sum_rows(dy * y) is added to dgain
  float* dgain;         // fp32 [2D]
  float* dq_acc;        // NULL, or workspace fp32 [2][B*H][n_pad][64]: partial sums of dQ1, dQ2 of the single-pass kernel
                        // (bwd_fused64.cuh); zeroed by the preprocess kernel, converted by the finishing kernel
  long long dq_acc_f4;  // its size in float4 units
};

// Row statistics, interleaved by pairs of rows so that a kernel that walks two neighbouring rows (the key-side
// kernels: two query columns of a thread's 16) gets each quantity of both rows in one 64-bit register pair, the
// operand form of the packed fp32 instructions: rows 2q and 2q+1 occupy floats
//   [8q .. 8q+8) = { x(2q), x(2q+1), y(2q), y(2q+1), z(2q), z(2q+1), w(2q), w(2q+1) }.
// idx = (batch*head) * n_pad + row; n_pad is even, so a pair never straddles two heads.
__device__ __forceinline__ void stat_store(float4* stats, long long idx, float4 v) {
  float* f = reinterpret_cast<float*>(stats + (idx & ~1ll)) + (idx & 1);
  f[0] = v.x; f[2] = v.y; f[4] = v.z; f[6] = v.w;
}
__device__ __forceinline__ float4 stat_row(const float4* stats, size_t idx) {
  const float* f = reinterpret_cast<const float*>(stats + (idx & ~size_t(1))) + (idx & 1);
  return make_float4(f[0], f[2], f[4], f[6]);
}

// ------------------------------------------------------------------------------------------------
// 1. preprocess: one warp per row, DV = 32 * VPL halves per row
// ------------------------------------------------------------------------------------------------
template <int VPL, bool BF>   // 16-bit elements per lane: 2 (DV=64), 4 (DV=128), 8 (DV=256); BF: bf16 tensors
__global__ void __launch_bounds__(256) diffattn_bwd_pre_kernel(const BwdArgs args) {
  // rows per warp and trip (see below).  Measured at B4 H16 N4096 D64: 1 / 2 / 3 / 4 / 8 rows 0.103 / 0.072 / 0.078 / 0.093 /
  // 0.089 ms (two rows keep the kernel at 63 registers, four resident CTAs per SM); at D = 128 and D = 32 four rows are
  // as good or better (0.062 ms each).
  constexpr int PRE_ROWS = VPL == 4 ? 2 : 4;
  constexpr int DV = 32 * VPL;
  constexpr float LOG2E = 1.4426950408889634f;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long warps_total = (long long)gridDim.x * (blockDim.x >> 5);
  const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
  const float c = args.out_scale;
  float dl_acc = 0.f;
  __shared__ float red[8];
  // learnable gain of the output norm: Y_out = Y * gain, so dY = dY_out * gain and d(gain) = sum over rows of dY_out * Y
  const bool has_gain = args.gain != nullptr;
  float gn[VPL], dg_acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) { gn[i] = has_gain ? args.gain[lane * VPL + i] : 1.f; dg_acc[i] = 0.f; }
  __shared__ float dg_red[8][DV];
  // the dQ partial sums of the single-pass backward start from zero
  if (args.dq_acc) {
    float4* z = reinterpret_cast<float4*>(args.dq_acc);
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < args.dq_acc_f4; t += (long long)gridDim.x * blockDim.x)
      z[t] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // PRE_ROWS rows per warp and trip: all their loads are issued before the first reduction, which keeps that many
  // times the bytes in flight per warp (one row per trip ran at 26 % of the DRAM rate: the shuffles of a row's two
  // reductions sat between its loads and the next row's).
  const long long first = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  for (long long row0 = first; row0 < args.rows; row0 += warps_total * PRE_ROWS) {
    __align__(16) __half hdr[PRE_ROWS][VPL], hyr[PRE_ROWS][VPL], har[PRE_ROWS][VPL];
    float rsr[PRE_ROWS], l1r[PRE_ROWS], l2r[PRE_ROWS];
#pragma unroll
    for (int rr = 0; rr < PRE_ROWS; ++rr) {
      const long long row = row0 + rr * warps_total;
      if (row < args.rows) {
        const size_t off = size_t(row) * DV + lane * VPL;
        __half* hd = hdr[rr]; __half* hy = hyr[rr]; __half* ha = har[rr];
        if constexpr (VPL == 8) {
          *reinterpret_cast<uint4*>(hd) = *reinterpret_cast<const uint4*>(args.dy + off);
          *reinterpret_cast<uint4*>(hy) = *reinterpret_cast<const uint4*>(args.y + off);
          *reinterpret_cast<uint4*>(ha) = *reinterpret_cast<const uint4*>(args.a2 + off);
        } else if constexpr (VPL == 4) {
          *reinterpret_cast<uint2*>(hd) = *reinterpret_cast<const uint2*>(args.dy + off);
          *reinterpret_cast<uint2*>(hy) = *reinterpret_cast<const uint2*>(args.y + off);
          *reinterpret_cast<uint2*>(ha) = *reinterpret_cast<const uint2*>(args.a2 + off);
        } else {
          *reinterpret_cast<uint32_t*>(hd) = *reinterpret_cast<const uint32_t*>(args.dy + off);
          *reinterpret_cast<uint32_t*>(hy) = *reinterpret_cast<const uint32_t*>(args.y + off);
          *reinterpret_cast<uint32_t*>(ha) = *reinterpret_cast<const uint32_t*>(args.a2 + off);
        }
        rsr[rr] = args.rstd[row]; l1r[rr] = args.lse1[row]; l2r[rr] = args.lse2[row];
      }
    }
#pragma unroll
    for (int rr = 0; rr < PRE_ROWS; ++rr) {      // (body kept at the indentation of the one-row loop it came from)
    const long long row = row0 + rr * warps_total;
    if (row >= args.rows) break;
    const size_t off = size_t(row) * DV + lane * VPL;
    const __half* hd = hdr[rr]; const __half* hy = hyr[rr]; const __half* ha = har[rr];
    float dy[VPL], yv[VPL], a2[VPL];
    {
#pragma unroll
      for (int i = 0; i < VPL; ++i) { dy[i] = to_float16b<BF>(hd[i]); yv[i] = to_float16b<BF>(hy[i]); a2[i] = to_float16b<BF>(ha[i]); }
    }
    if (has_gain) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) { dg_acc[i] = fmaf(dy[i], yv[i], dg_acc[i]); dy[i] *= gn[i]; }
    }
    float da[VPL], av[VPL];
    if (args.rms_norm) {
      // Y = c r A  =>  A = Y/(c r),  dA = r (c dY - Y (dY.Y) / (c Dv));  c == 0 gives dA = 0
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) t += dy[i] * yv[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      const float r = rsr[rr];
      const float inv_c = c != 0.f ? 1.f / c : 0.f;
      const float k1 = r * c, k2 = r * inv_c * t * (1.f / DV), k3 = inv_c / r;
#pragma unroll
      for (int i = 0; i < VPL; ++i) { da[i] = k1 * dy[i] - k2 * yv[i]; av[i] = yv[i] * k3; }
    } else {
#pragma unroll
      for (int i = 0; i < VPL; ++i) { da[i] = dy[i]; av[i] = yv[i]; }
    }
    // round dA to the 16-bit type first: the row sums below must agree with what the MMAs will see
    __half hda[VPL];
    float e2 = 0.f, ea = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      hda[i] = from_float16b<BF>(da[i]);
      const float d = to_float16b<BF>(hda[i]);
      e2 += d * a2[i];
      ea += d * av[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      e2 += __shfl_xor_sync(0xffffffffu, e2, o);
      ea += __shfl_xor_sync(0xffffffffu, ea, o);
    }
    if constexpr (VPL == 8) *reinterpret_cast<uint4*>(args.da + off) = *reinterpret_cast<uint4*>(hda);
    else if constexpr (VPL == 4) *reinterpret_cast<uint2*>(args.da + off) = *reinterpret_cast<uint2*>(hda);
    else *reinterpret_cast<uint32_t*>(args.da + off) = *reinterpret_cast<uint32_t*>(hda);
    if (lane == 0) {
      // E1 - lam E2 = rowsum(dA * A).  lambda is folded into the branch-2 statistics so that the tensor-core
      // kernels need no multiply for it: with P2' = |lam| P2 = 2^(s S2 log2e - y) and sg = -sign(lam),
      // -lam P2 = sg P2' and -lam P2 (dP - E2) = P2' (sg dP - w).  lam = 0 gives y = +inf, P2' = 0.
      const float sg = lam < 0.f ? 1.f : -1.f;
      const long long bh_i = row / args.n;
      stat_store(args.stats, bh_i * args.n_pad + (row - bh_i * args.n),
                 make_float4(-l1r[rr] * LOG2E, log2f(fabsf(lam)) - l2r[rr] * LOG2E, -(ea + lam * e2), -sg * e2));
      dl_acc -= e2;
    }
  }
  }
  if (lane == 0) red[warp] = dl_acc;
  if (has_gain) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) dg_red[warp][lane * VPL + i] = dg_acc[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
    atomicAdd(args.dlambda, s);
  }
  if (has_gain && threadIdx.x < DV) {
    float s = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) s += dg_red[i][threadIdx.x];
    atomicAdd(args.dgain + threadIdx.x, s);       // one atomic per column and CTA
  }
}

// rows N..n_pad-1 of every (batch, head) in `stats`: neutral values (see BwdArgs::n_pad)
__global__ void diffattn_bwd_padstats_kernel(const BwdArgs args, int bh_total) {
  const int pad = args.n_pad - args.n;
  const long long total = (long long)bh_total * pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long bh_i = i / pad;
    stat_store(args.stats, bh_i * args.n_pad + args.n + (i - bh_i * pad), make_float4(-INFINITY, -INFINITY, 0.f, 0.f));
  }
}

// ------------------------------------------------------------------------------------------------
// 2. dK1, dK2, dV: one CTA = 128 key/value rows of one (batch, head); query tiles of 64 stream by.
// TMEM: dV [0,128) dK1 [128,192) dK2 [192,256) | scores S1^T [256,320) S2^T [320,384) dP^T [384,448) |
// fp16 A-operands dS1^T [448,480) dS2^T [480,512).  Thread = key row; four warpgroups, warpgroup g handles
// query columns [16g, 16g+16) (more resident warps per scheduler hide the exp-unit and TMEM latencies).  The warpgroups pull their scores into registers and release the score columns at once,
// so the MMAs of tile i+1 run under the elementwise work of tile i.  dS_b^T goes back to TMEM (A-operand of
// dK_b += dS_b^T Q_b); (P1 - lam P2)^T goes to a double-buffered K-major shared-memory tile (A-operand of
// dV += Pc^T dA) because TMEM has no columns left for it.
// ------------------------------------------------------------------------------------------------
// Per-column statistics are read from shared memory DA_PF columns ahead of their use, by volatile loads that keep
// that order: every thread of a warp reads the same 16 bytes per column, and left to the compiler the loads sat
// right before their consumers with the shared-memory pipe's loaded latency exposed 16 times per tile (at
// B4 H16 N4096 D64 the dK/dV kernel took 1.33 ms that way; 1.22 ms with two columns ahead, 1.23 with four).
#ifndef DA_PF
#define DA_PF 2
#endif
__device__ __forceinline__ float4 lds_v4(const float4* p) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)));
  return v;
}
namespace dkdv64 {
// (ring depth 4 with a single Pc buffer, and depth 3 with a single buffer, measured within noise of this setting)
constexpr int BKV = 128, BQ = 64, HD = 64, DV = 128, ST = 3, PCBUF = 2;
constexpr int K_BYTES = BKV * HD * 2;       // 16 KB
constexpr int V_BYTES = BKV * DV * 2;       // 32 KB, two boxes of 16 KB
constexpr int Q_BYTES = BQ * HD * 2;        // 8 KB
constexpr int DA_BYTES = BQ * DV * 2;       // 16 KB, two boxes of 8 KB
constexpr int STAT_BYTES = BQ * 16;         // 1 KB
constexpr int STAGE_BYTES = 2 * Q_BYTES + DA_BYTES + STAT_BYTES;   // 33 KB
constexpr int PC_BYTES = BKV * BQ * 2;      // 16 KB per buffer
constexpr int OFF_K1 = 0, OFF_K2 = K_BYTES, OFF_V = 2 * K_BYTES;
constexpr int OFF_PC = OFF_V + V_BYTES;                            // 64 KB
constexpr int OFF_STAGE = OFF_PC + PCBUF * PC_BYTES;                   // 96 KB
constexpr int OFF_MISC = OFF_STAGE + ST * STAGE_BYTES;             // 195 KB
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int NWG = 4;                      // elementwise warpgroups; warpgroup g owns query columns [16g, 16g+16)
constexpr int NUM_THREADS = NWG * 128 + 128;                      // + TMA warp and three MMA-issuing warps, one per scheduler
constexpr int WARP_TMA = NWG * 4, WARP_MMA = NWG * 4 + 1;         // issuers: WARP_MMA (S^T), +1 (dP^T), +2 (dV, dK)
constexpr int T_DV = 0, T_DK1 = 128, T_DK2 = 192, T_S1 = 256, T_S2 = 320, T_DP = 384, T_DS1 = 448, T_DS2 = 480;
struct Misc {
  uint64_t bar_kv;
  uint64_t full[ST], empty[ST];
  uint64_t s_full;      // scores of a tile written (MMA -> warpgroups)
  uint64_t s_free;      // scores of a tile are in registers (one arrival per elementwise thread)
  uint64_t e_done;      // dS^T in TMEM and Pc in shared memory written (one arrival per elementwise thread)
  uint64_t mma_done;    // dV/dK MMAs of a tile completed (operand buffers reusable)
  uint64_t acc_full;
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace dkdv64

template <bool BF, bool DROP>
__global__ void __launch_bounds__(dkdv64::NUM_THREADS, 1)
diffattn_bwd_dkdv64_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                           const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_da,
                           const __grid_constant__ CUtensorMap tm_dk1, const __grid_constant__ CUtensorMap tm_dk2,
                           const __grid_constant__ CUtensorMap tm_dv, const BwdArgs args) {
  using namespace dkdv64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, bh = blockIdx.y;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  // the last query tiles may reach past N (zero dA, neutral statistics); under the causal mask only query tiles
  // from the diagonal on see these keys: tiles i0 .. nq_all-1, visited with the local index i (tile i0 + i)
  const int nq_all = args.n_pad / BQ;
  const int i0 = args.causal ? kv_tile * (BKV / BQ) : 0;
  const int nq = nq_all - i0;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_kv, 1);
    for (int i = 0; i < ST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->empty[i], 1); }
    mbar_init(&misc->s_full, 2);
    mbar_init(&misc->s_free, NWG * 128);
    mbar_init(&misc->e_done, NWG * 128);
    mbar_init(&misc->mma_done, 1);
    mbar_init(&misc->acc_full, 1);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == WARP_MMA) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  // (Requesting the resident tiles and the first ring pass before the setup barrier, as the forward and the dQ
  // kernel do, measured 3 % slower here.)
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
        if (!mbar_wait(&misc->empty[st], ((i / ST) & 1) ^ 1, abort_flag, 401, i)) break;
        mbar_expect_tx(&misc->full[st], STAGE_BYTES);
        tma_load_4d(sp, &tm_q1, &misc->full[st], 0, (i0 + i) * BQ, h_idx, b_idx);
        tma_load_4d(sp + Q_BYTES, &tm_q2, &misc->full[st], 0, (i0 + i) * BQ, h_idx, b_idx);
        tma_load_4d(sp + 2 * Q_BYTES, &tm_da, &misc->full[st], 0, (i0 + i) * BQ, bh, 0);
        tma_load_4d(sp + 2 * Q_BYTES + DA_BYTES / 2, &tm_da, &misc->full[st], 64, (i0 + i) * BQ, bh, 0);
        bulk_load_1d(sp + 2 * Q_BYTES + DA_BYTES, args.stats + (size_t(bh) * args.n_pad + size_t(i0 + i) * BQ), STAT_BYTES,
                     &misc->full[st]);
      }
    }
  } else if (warp == WARP_MMA || warp == WARP_MMA + 1) {
    // ---- score issuers: warp WARP_MMA issues S1^T and S2^T of every tile, warp WARP_MMA + 1 issues dP^T.
    // MMA issue is spread over three warps on three schedulers (these two and the output issuer below): one warp
    // issuing all 32 MMAs of a tile takes ~300 clocks per tile from the elementwise warps of its scheduler, and
    // every tile waits for that slowest quarter.  One elected thread per warp; descriptors advance by 32-bit adds.
    if (elect_one()) {
      const bool is_dp = warp == WARP_MMA + 1;
      constexpr uint32_t IDESC_S = make_idesc(BKV, BQ, 0, 0, BF);     // S^T = K Q^T, dP^T = V dA^T
      const uint32_t k1_lo = sdesc_lo(smem_u32(smem + OFF_K1)), k2_lo = sdesc_lo(smem_u32(smem + OFF_K2));
      const uint32_t v_lo = sdesc_lo(smem_u32(smem + OFF_V));
      const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
      const uint32_t tb = tmem_base;
      const int kd = args.d >> 4;       // 16-deep MMA steps over the head dim (value width: twice as many): head dim 32 skips the zero padding
      auto issue_scores = [&](uint32_t sp_lo) {
        if (!is_dp) {
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)
            if (k < kd) mma_ss_lo(tb + T_S1, k1_lo + k * 2, sp_lo + k * 2, IDESC_S, k > 0);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k)
            if (k < kd) mma_ss_lo(tb + T_S2, k2_lo + k * 2, sp_lo + (Q_BYTES >> 4) + k * 2, IDESC_S, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < DV / 16; ++k)
            if (k < 2 * kd)
              mma_ss_lo(tb + T_DP, v_lo + (k / 4) * ((V_BYTES / 2) >> 4) + (k % 4) * 2,
                        sp_lo + ((2 * Q_BYTES) >> 4) + (k / 4) * ((DA_BYTES / 2) >> 4) + (k % 4) * 2, IDESC_S, k > 0);
        }
        mma_commit(&misc->s_full);        // two arrivals per tile: this warp's and the other score issuer's
      };
      bool ok = mbar_wait(&misc->bar_kv, 0, abort_flag, 501);
      ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 502);
      if (ok) {
        tc_fence_after();
        issue_scores(st_lo0);
        int st = 0;
        uint32_t st_par = 0;
        for (int i = 0; i + 1 < nq; ++i) {
          int st_n = st + 1;
          uint32_t par_n = st_par;
          if (st_n == ST) { st_n = 0; par_n ^= 1; }
          if (!mbar_wait(&misc->full[st_n], par_n, abort_flag, 503, i)) break;
          if (!mbar_wait(&misc->s_free, i & 1, abort_flag, 504, i)) break;    // scores(i) are in registers
          tc_fence_after();
          issue_scores(st_lo0 + st_n * (STAGE_BYTES >> 4));
          st = st_n;
          st_par = par_n;
        }
      }
    }
  } else if (warp == WARP_MMA + 2) {
    // ---- output issuer: dV += Pc^T dA, dK_b += dS_b^T Q_b of tile i once the warpgroups have written their operands
    if (elect_one()) {
      // head dim 32: only the real 64 value columns / 32 head columns are produced
      const uint32_t IDESC_DV = make_idesc(BKV, 2 * args.d, 0, 1, BF);    // dV += Pc^T dA   (Pc K-major smem, dA MN-major)
      const uint32_t IDESC_DK = make_idesc(BKV, args.d, 0, 1, BF);        // dK += dS^T Q    (dS^T in TMEM, Q MN-major)
      const uint32_t pc_lo0 = sdesc_lo(smem_u32(smem + OFF_PC));
      const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
      constexpr uint32_t DA_MN_LBO = ((DA_BYTES / 2) >> 4) << 16;   // dA as MN-major B: 64-column atoms 8 KB apart
      const uint32_t tb = tmem_base;
      int st = 0;
      for (int i = 0; i < nq; ++i) {
        const uint32_t sp_lo = st_lo0 + st * (STAGE_BYTES >> 4);
        const uint32_t pc_lo = pc_lo0 + (i % PCBUF) * (PC_BYTES >> 4);
        // e_done(i) implies that stage i was loaded and that the score MMAs reading it have completed
        if (!mbar_wait(&misc->e_done, i & 1, abort_flag, 505, i)) break;
        tc_fence_after();
        const uint32_t first = i > 0;
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          mma_ss_lo(tb + T_DV, pc_lo + k * 2, sp_lo + ((2 * Q_BYTES) >> 4) + DA_MN_LBO - (1u << 16) + k * (2048 >> 4), IDESC_DV,
                    k > 0 ? 1u : first);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          mma_ts_lo(tb + T_DK1, tb + T_DS1 + k * 8, sp_lo + k * (2048 >> 4), IDESC_DK, k > 0 ? 1u : first);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)
          mma_ts_lo(tb + T_DK2, tb + T_DS2 + k * 8, sp_lo + (Q_BYTES >> 4) + k * (2048 >> 4), IDESC_DK, k > 0 ? 1u : first);
        mma_commit(&misc->mma_done);
        mma_commit(&misc->empty[st]);
        if (++st == ST) st = 0;
      }
      mma_commit(&misc->acc_full);
    }
  } else {
    const int g = warp >> 2;                       // warpgroup: query columns [16g, 16g+16) of every tile
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tb = tmem_base + lane_base;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const float sg = load_lambda(args.lambda_ptr, args.lambda_dtype) < 0.f ? 1.f : -1.f;   // -sign(lambda)
    // dropout: this thread owns key column kv_tile*BKV + row; a hash covers two consecutive query rows of it
    const uint32_t dkey1 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 0u) : 0u;
    const uint32_t dkey2 = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), 1u) : 0u;
    const uint32_t dcol2 = uint32_t(kv_tile * BKV + row) >> 1;
    const int dcol_odd = row & 1;
    const float dscale = DROP ? args.drop_scale : 1.f;
    const f32x2 sl2_2 = pk2(sl2, sl2), sg_2 = pk2(sg, sg);
    bool ok = true;
    uint32_t s_ready = 0;            // answers of the early probes (see mbar_probe)
    for (int i = 0; i < nq; ++i) {
      const int st = i % ST;
      const float4* stats = reinterpret_cast<const float4*>(smem + OFF_STAGE + st * STAGE_BYTES + 2 * Q_BYTES + DA_BYTES) + g * 16;
      if (!s_ready && !mbar_wait(&misc->s_full, i & 1, abort_flag, 601 + g, i)) { ok = false; break; }
      tc_fence_after();
      uint32_t s1[16], s2[16], dp[16];
      tmem_ld16(tb + T_S1 + g * 16, s1);
      tmem_ld16(tb + T_S2 + g * 16, s2);
      tmem_ld16(tb + T_DP + g * 16, dp);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&misc->s_free);
      if (args.causal) {
        // this thread's key row sees query columns >= its own index only: the first c0 columns of its 16 are hidden
        const int c0 = kv_tile * BKV + row - ((i0 + i) * BQ + g * 16);
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
          const uint32_t drow2 = uint32_t((i0 + i) * (BQ / 2) + g * 8 + jj);
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
      // The dS^T columns are free once the output MMAs of tile i-1 have completed (mma_done); the Pc buffer of this
      // tile was last read by tile i-2, whose completion the previous trip waited for.  So the Pc stores and their
      // proxy fence go first, under the latency of an early look at mma_done (see mbar_probe).
      static_assert(PCBUF == 2, "the Pc buffer of tile i must be the one tile i-2 used");
      const uint32_t md_ready = i > 0 ? mbar_probe(&misc->mma_done, (i - 1) & 1) : 1u;
      // Pc tile [128 key rows][64 query columns] fp16, 128-byte rows, 16-byte chunks XOR-swizzled by row
      {
        uint8_t* prow = smem + OFF_PC + (i % PCBUF) * PC_BYTES + row * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int chunk = (g * 2 + c) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pc[4 * c], pc[4 * c + 1], pc[4 * c + 2], pc[4 * c + 3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (i > 0) {
        if (!md_ready && !mbar_wait(&misc->mma_done, (i - 1) & 1, abort_flag, 605 + g, i)) { ok = false; break; }
        tc_fence_after();
      }
      s_ready = i + 1 < nq ? mbar_probe(&misc->s_full, (i + 1) & 1) : 0u;
      // 8 packed columns per warpgroup: the 32x32b.x8 shape
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                   ::"r"(tb + T_DS1 + g * 8), "r"(d1[0]), "r"(d1[1]), "r"(d1[2]), "r"(d1[3]), "r"(d1[4]), "r"(d1[5]), "r"(d1[6]), "r"(d1[7]) : "memory");
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                   ::"r"(tb + T_DS2 + g * 8), "r"(d2[0]), "r"(d2[1]), "r"(d2[2]), "r"(d2[3]), "r"(d2[4]), "r"(d2[5]), "r"(d2[6]), "r"(d2[7]) : "memory");
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->e_done);
    }
    ok = ok && mbar_wait(&misc->acc_full, 0, abort_flag, 611 + g);
    tc_fence_after();
    // warpgroup g reads accumulator columns [64g, 64g+64): g = 0,1 -> the two halves of dV, g = 2 -> dK1, g = 3 -> dK2
    uint32_t acc[64];
    tmem_ld32(tb + g * 64, acc);
    tmem_ld32(tb + g * 64 + 32, acc + 32);
    tc_wait_ld();
    // The gradients leave through shared memory and the TMA engine (row-per-thread global stores of 16-byte
    // pieces are several times slower): each warpgroup lays its 64 columns into a swizzled [128][64] tile over
    // the resident K1 / K2 / V tiles, which no MMA reads any more, and one of its threads stores the tile.
    // The engine clips at the tensor's bounds: key rows past the sequence end and, for head dim 32, the
    // padding columns are not written.
    {
      const float s = g < 2 ? 1.f : args.sm_scale;
      uint8_t* tile = smem + ((g + 2) & 3) * K_BYTES;     // g = 0,1 -> the two halves of V; 2 -> K1; 3 -> K2
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 v;
        v.x = pack2<BF>(__uint_as_float(acc[8 * i + 0]) * s, __uint_as_float(acc[8 * i + 1]) * s);
        v.y = pack2<BF>(__uint_as_float(acc[8 * i + 2]) * s, __uint_as_float(acc[8 * i + 3]) * s);
        v.z = pack2<BF>(__uint_as_float(acc[8 * i + 4]) * s, __uint_as_float(acc[8 * i + 5]) * s);
        v.w = pack2<BF>(__uint_as_float(acc[8 * i + 6]) * s, __uint_as_float(acc[8 * i + 7]) * s);
        st_swizzled_chunk(tile, row, i, v);
      }
      fence_proxy_async_smem();
      named_bar_sync(1 + g, 128);
      const int dv_real = 2 * args.d;
      if ((warp & 3) == 0 && elect_one()) {
        if (!*abort_flag && (g != 1 || dv_real > 64)) {
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
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// 3. dQ1, dQ2: one CTA = 128 query rows; key/value tiles of 128 rows stream by and are consumed in
// sub-tiles of 64 rows.  TMEM: S1 two 64-column buffers [0,128), S2 [128,256), dP [256,384),
// dQ1 [384,448), dQ2 [448,512).  Thread = query row; four warpgroups: two per branch, each forming
// dS_b = +-P_b (dP - E_b) for 32 of the 64 columns of a sub-tile and writing it as fp16 over the first 16 of its
// own columns (TMEM A-operand of dS_b K_b).  The MMAs of sub-tile t+1 are issued before
// the issuer waits for dS(t), so the warpgroups always find their next scores ready.
// ------------------------------------------------------------------------------------------------
// (Separate ring barriers for the V part of a stage, free half a tile before the K part, measured no change here:
// this kernel does not wait for its loads.  The D = 128 kernels did, see bwd128.cuh.)
namespace dq64 {
constexpr int BM = 128, BN = 128, SUB = 64, HD = 64, DV = 128, ST = 2;
constexpr int Q_BYTES = BM * HD * 2;        // 16 KB
constexpr int DA_BYTES = BM * DV * 2;       // 32 KB
constexpr int K_BYTES = BN * HD * 2;        // 16 KB
constexpr int V_BYTES = BN * DV * 2;        // 32 KB
constexpr int STAGE_BYTES = 2 * K_BYTES + V_BYTES;   // 64 KB
constexpr int OFF_Q1 = 0, OFF_Q2 = Q_BYTES, OFF_DA = 2 * Q_BYTES;
constexpr int OFF_STAGE = OFF_DA + DA_BYTES;         // 64 KB
constexpr int OFF_MISC = OFF_STAGE + ST * STAGE_BYTES;
constexpr int MISC_BYTES = 1024;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int NWG = 4;                      // warpgroup w: branch w>>1, columns [32(w&1), 32(w&1)+32) of each sub-tile
constexpr int NUM_THREADS = NWG * 128 + 64;
constexpr int WARP_TMA = NWG * 4, WARP_MMA = NWG * 4 + 1;
constexpr int T_S1 = 0, T_S2 = 128, T_DP = 256, T_DQ1 = 384, T_DQ2 = 448;
struct Misc {
  uint64_t bar_q;
  uint64_t full[ST], empty[ST];
  uint64_t s_full[2][2], ds_full[2][2], acc_full;   // [branch][buffer]
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace dq64

template <bool BF, bool DROP>
__global__ void __launch_bounds__(dq64::NUM_THREADS, 1)
diffattn_bwd_dq64_kernel(const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_q2,
                         const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_k2,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_da,
                         const BwdArgs args) {
  using namespace dq64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Misc* misc = reinterpret_cast<Misc*>(smem + OFF_MISC);
  volatile int* abort_flag = &misc->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the later a query tile, the more keys it sees -- the heaviest tiles are launched first so that the grid's tail is light
  const int q_tile = args.causal ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x), bh = blockIdx.y;
  const int b_idx = bh / args.h, h_idx = bh % args.h;
  const int nkv_all = args.n_pad / BN;
  const int nkv = (args.causal && q_tile + 1 < nkv_all) ? q_tile + 1 : nkv_all;   // causal: stop at the diagonal tile
  const int nsub = 2 * nkv;

  if (warp == WARP_TMA && lane == 0) {
    mbar_init(&misc->bar_q, 1);
    for (int i = 0; i < ST; ++i) { mbar_init(&misc->full[i], 1); mbar_init(&misc->empty[i], 1); }
    for (int b = 0; b < 2; ++b)
      for (int u = 0; u < 2; ++u) { mbar_init(&misc->s_full[b][u], 1); mbar_init(&misc->ds_full[b][u], 256); }
    mbar_init(&misc->acc_full, 1);
    misc->abort_flag = 0;
    mbar_init_fence();
  }
  // key/value stage j (tile j) into ring slot j % ST
  auto load_stage = [&](int j) {
    const int st = j % ST;
    uint8_t* sp = smem + OFF_STAGE + st * STAGE_BYTES;
    mbar_expect_tx(&misc->full[st], STAGE_BYTES);
    tma_load_4d(sp, &tm_k1, &misc->full[st], 0, j * BN, h_idx, b_idx);
    tma_load_4d(sp + K_BYTES, &tm_k2, &misc->full[st], 0, j * BN, h_idx, b_idx);
    tma_load_4d(sp + 2 * K_BYTES, &tm_v, &misc->full[st], 0, j * BN, h_idx, b_idx);
    tma_load_4d(sp + 2 * K_BYTES + V_BYTES / 2, &tm_v, &misc->full[st], 64, j * BN, h_idx, b_idx);
  };
  if (warp == WARP_TMA && lane == 0) {
    // the resident tiles and the first pass over the ring are requested before the CTA-wide setup barrier
    mbar_expect_tx(&misc->bar_q, 2 * Q_BYTES + DA_BYTES);
    tma_load_4d(smem + OFF_Q1, &tm_q1, &misc->bar_q, 0, q_tile * BM, h_idx, b_idx);
    tma_load_4d(smem + OFF_Q2, &tm_q2, &misc->bar_q, 0, q_tile * BM, h_idx, b_idx);
    tma_load_4d(smem + OFF_DA, &tm_da, &misc->bar_q, 0, q_tile * BM, bh, 0);
    tma_load_4d(smem + OFF_DA + DA_BYTES / 2, &tm_da, &misc->bar_q, 64, q_tile * BM, bh, 0);
    for (int j = 0; j < ST && j < nkv; ++j) load_stage(j);
  }
  if (warp == WARP_MMA) tmem_alloc(&misc->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&misc->tmem_slot);

  if (warp == WARP_TMA) {
    if (elect_one()) {
      for (int j = ST; j < nkv; ++j) {
        if (!mbar_wait(&misc->empty[j % ST], ((j / ST) & 1) ^ 1, abort_flag, 701, j)) break;
        load_stage(j);
      }
    }
  } else if (warp == WARP_MMA) {
    // One elected thread issues every MMA; descriptors advance by 32-bit adds (see sm100.cuh).  (Three issuing warps
    // as in the dK/dV kernel were measured here in two forms: split by kind (S | dP | dQ, which needs a committed
    // mbarrier between the dQ and the S issuer because the score buffers are recycled on the tensor pipe's issue
    // order): 1.00 against 0.92 ms; split by branch (S_b and dQ_b | dP, which keeps that order): 0.98 ms.  Both
    // slower: the single issuer stays.  So did two issuing warps, one per branch (S_b and dQ_b, dP of alternate sub-tiles,
    // no barrier between the two): 0.944 against 0.912 ms -- although the elementwise warps that share a scheduler with
    // the single issuer finish every sub-tile 130-300 clocks after the others.)
    if (elect_one()) {
      constexpr uint32_t IDESC_S = make_idesc(BM, SUB, 0, 0, BF);    // S = Q K^T, dP = dA V^T
      const uint32_t IDESC_DQ = make_idesc(BM, args.d, 0, 1, BF);    // dQ += dS K   (K MN-major); head dim 32: 32 columns
      const int kd = args.d >> 4;       // 16-deep MMA steps over the head dim: head dim 32 skips the zero padding
      constexpr uint32_t HALF = (SUB * 128) >> 4;
      const uint32_t q1_lo = sdesc_lo(smem_u32(smem + OFF_Q1)), q2_lo = sdesc_lo(smem_u32(smem + OFF_Q2));
      const uint32_t da_lo = sdesc_lo(smem_u32(smem + OFF_DA));
      const uint32_t st_lo0 = sdesc_lo(smem_u32(smem + OFF_STAGE));
      const uint32_t tb = tmem_base;
      // scores of a 64-row sub-tile into buffer u: S1 and dP (commit -> branch 1), then S2 (commit -> branch 2)
      auto issue_scores = [&](uint32_t sp_lo, int u) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          if (k < kd) mma_ss_lo(tb + T_S1 + u * SUB, q1_lo + k * 2, sp_lo + u * HALF + k * 2, IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)
          if (k < 2 * kd)
            mma_ss_lo(tb + T_DP + u * SUB, da_lo + (k / 4) * ((DA_BYTES / 2) >> 4) + (k % 4) * 2,
                      sp_lo + ((2 * K_BYTES) >> 4) + (k / 4) * ((V_BYTES / 2) >> 4) + u * HALF + (k % 4) * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[0][u]);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          if (k < kd) mma_ss_lo(tb + T_S2 + u * SUB, q2_lo + k * 2, sp_lo + (K_BYTES >> 4) + u * HALF + k * 2, IDESC_S, k > 0);
        mma_commit(&misc->s_full[1][u]);
      };
      auto issue_dq = [&](int br, uint32_t sp_lo, int u, uint32_t first) {
#pragma unroll
        for (int k = 0; k < SUB / 16; ++k)
          mma_ts_lo(tb + (br ? T_DQ2 : T_DQ1), tb + (br ? T_S2 : T_S1) + u * SUB + (k / 2) * 32 + (k % 2) * 8,
                    sp_lo + br * (K_BYTES >> 4) + u * HALF + k * (2048 >> 4), IDESC_DQ, k > 0 ? 1u : first);
      };
      bool ok = mbar_wait(&misc->bar_q, 0, abort_flag, 801);
      ok = ok && mbar_wait(&misc->full[0], 0, abort_flag, 802);
      if (ok) {
        tc_fence_after();
        issue_scores(st_lo0, 0);
        int st = 0;
        uint32_t st_par = 0;
        for (int j = 0; j < nkv; ++j) {
          const uint32_t sp_lo = st_lo0 + st * (STAGE_BYTES >> 4);
          const uint32_t ph = j & 1;
          int st_n = st + 1;
          uint32_t par_n = st_par;
          if (st_n == ST) { st_n = 0; par_n ^= 1; }
          // ---- sub-tile 2j (buffer 0): scores of 2j+1 first
          issue_scores(sp_lo, 1);
          if (!mbar_wait(&misc->ds_full[0][0], ph, abort_flag, 804, j)) break;
          tc_fence_after();
          issue_dq(0, sp_lo, 0, j > 0);
          if (!mbar_wait(&misc->ds_full[1][0], ph, abort_flag, 805, j)) break;
          tc_fence_after();
          issue_dq(1, sp_lo, 0, j > 0);
          // ---- sub-tile 2j+1 (buffer 1): scores of 2j+2 (next tile) first
          if (j + 1 < nkv) {
            if (!mbar_wait(&misc->full[st_n], par_n, abort_flag, 803, j)) break;
            tc_fence_after();
            issue_scores(st_lo0 + st_n * (STAGE_BYTES >> 4), 0);
          }
          if (!mbar_wait(&misc->ds_full[0][1], ph, abort_flag, 806, j)) break;
          tc_fence_after();
          issue_dq(0, sp_lo, 1, 1);
          if (!mbar_wait(&misc->ds_full[1][1], ph, abort_flag, 807, j)) break;
          tc_fence_after();
          issue_dq(1, sp_lo, 1, 1);
          mma_commit(&misc->empty[st]);
          st = st_n;
          st_par = par_n;
        }
        mma_commit(&misc->acc_full);
      }
    }
  } else {
    const int br = warp >> 3;                      // branch
    const int half = (warp >> 2) & 1;              // which 32 of the 64 columns of a sub-tile
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tb = tmem_base + lane_base;
    const float sl2 = args.sm_scale * 1.4426950408889634f;
    const float lam = load_lambda(args.lambda_ptr, args.lambda_dtype);
    const size_t grow = size_t(bh) * args.n + size_t(q_tile) * BM + row;
    const float4 sv = stat_row(args.stats, size_t(bh) * args.n_pad + size_t(q_tile) * BM + row);
    const float neg_l = br ? sv.y : sv.x;
    const float neg_e = br ? sv.w : sv.z;
    const float sg = (br && !(lam < 0.f)) ? -1.f : 1.f;      // branch 2: -sign(lambda) (|lambda| sits in neg_l, the sign in e)
    const uint32_t dkey = DROP ? drop_key(args.seed_lo, args.seed_hi, uint32_t(bh), uint32_t(br)) : 0u;
    const uint32_t drow2 = uint32_t(q_tile * BM + row) >> 1;
    const int drow_odd = row & 1;
    const float sgs = DROP ? sg * args.drop_scale : sg;
    const f32x2 sl2_2 = pk2(sl2, sl2), negl_2 = pk2(neg_l, neg_l), sg_2 = pk2(sg, sg), nege_2 = pk2(neg_e, neg_e);
    bool ok = true;
    for (int t = 0; t < nsub; ++t) {
      const int u = t & 1;
      // own 32 columns; the fp16 result goes to the first 16 of them (the other warpgroup's columns are untouched)
      const uint32_t t_s = tb + (br ? T_S2 : T_S1) + u * SUB + half * 32;
      const uint32_t t_dp = tb + T_DP + u * SUB + half * 32;
      if (!mbar_wait(&misc->s_full[br][u], (t >> 1) & 1, abort_flag, 901 + br, t)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[32], dp[32];
      tmem_ld32(t_s, s);
      tmem_ld32(t_dp, dp);
      tc_wait_ld();
      {
        // key columns past the sequence end or (causal) right of the diagonal: score -inf, probability 0
        const int c_first = t * SUB + half * 32;
        int nv = args.n - c_first;
        if (args.causal) nv = min(nv, q_tile * BM + row - c_first + 1);
        if (nv < 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= nv) s[i] = 0xff800000u;
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float x0, x1;
        up2(fma2(pk2u(s[2 * i], s[2 * i + 1]), sl2_2, negl_2), x0, x1);
        const float p0 = ex2(x0), p1 = ex2(x1);
        if constexpr (DROP) {
          // dP reaches a probability only where it was kept, with the factor 1/(1-p)
          const uint32_t hh = drop_hash(dkey, drow2, uint32_t(t * (SUB / 2) + half * 16 + i));
          const float g0 = drop_keep(hh, 2 * drow_odd, args.drop_thresh) ? sgs : 0.f;
          const float g1 = drop_keep(hh, 2 * drow_odd + 1, args.drop_thresh) ? sgs : 0.f;
          s[i] = pack2<BF>(p0 * fmaf(g0, __uint_as_float(dp[2 * i]), neg_e), p1 * fmaf(g1, __uint_as_float(dp[2 * i + 1]), neg_e));
        } else {
          float r0, r1;
          up2(mul2(pk2(p0, p1), fma2(pk2u(dp[2 * i], dp[2 * i + 1]), sg_2, nege_2)), r0, r1);
          s[i] = pack2<BF>(r0, r1);
        }
      }
      tmem_st16(t_s, s);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&misc->ds_full[br][u]);
    }
    ok = ok && mbar_wait(&misc->acc_full, 0, abort_flag, 911 + br);
    tc_fence_after();
    uint32_t acc[32];
    tmem_ld32(tb + (br ? T_DQ2 : T_DQ1) + half * 32, acc);
    tc_wait_ld();
    // (32 columns per thread: direct 16-byte stores; a shared-memory tile and a TMA store, as the other two
    // kernels use for their wider rows, measured 4 % slower here)
    if (ok && !*abort_flag && half * 32 < args.d && q_tile * BM + row < args.n) {
      const float sc = args.sm_scale;
      uint4* p = reinterpret_cast<uint4*>((br ? args.dq2 : args.dq1) + grow * args.d + half * 32);
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

}  // namespace da
