// Differential-attention forward for sm_100a: what the forward kernels share (arguments, tile geometry of the
// D <= 64 kernel).  The kernels themselves: fwd64.cuh (head dims 32 and 64), fwd128.cuh (head dim 128).
//
// One CTA owns one tile of 128 query rows of one (batch, head).  TMEM (512 columns of 128 lanes x 32 bit) at
// D <= 64: S1 two 64-column buffers [0,128), S2 likewise [128,256), O1 [256,384), O2 [384,512).  Scores are
// produced in sub-tiles of 64 key rows into alternating buffers, so the MMA for sub-tile t+1 runs while the
// softmax warps work on sub-tile t.  P_b (16-bit, two per column) overwrites the first 32 columns of its S
// buffer and is the TMEM A-operand of P_b V.
// Replaces the reference's Triton forward (src/kernel.py:21-207): same math (two online softmaxes,
// O = O1/l1 - lambda O2/l2, RMSNorm * (1 - lambda_init)), but saves lse1, lse2, rstd and A2 = P2 V
// instead of O1/O2.
#pragma once
#include "sm100.cuh"

namespace da {

struct FwdArgs {
  __half* y;          // [B*H, N, 2D] dense; "__half" stands for a 16-bit element here: fp16, or bf16 in the BF kernels
  __half* a2;         // [B*H, N, 2D] dense, branch-2 output P2 V (kept for the backward)
  float* lse1;        // [B*H, N] natural-log logsumexp of s Q1 K1^T
  float* lse2;
  float* rstd;        // [B*H, N] rsqrt(mean(A^2) + eps)   (written also when rms_norm is off)
  const void* lambda_ptr;
  int lambda_dtype;   // 0 = fp16, 1 = fp32, 2 = bf16
  float sm_scale;
  float out_scale;    // 1 - lambda_init
  float eps;
  int rms_norm;
  int n;              // sequence length
  int h;              // heads
  int d;              // real head dim: 64, or 32 (then the 64-wide tiles are zero-filled by TMA beyond column 32 / 64)
  int causal;         // 1: query row i sees key columns j <= i only
  uint32_t drop_thresh;   // dropout: 0 = off, else keep a probability iff its hash byte >= drop_thresh (see sm100.cuh)
  uint32_t seed_lo, seed_hi;
  float drop_scale;       // 256 / (256 - drop_thresh)
  const float* gain;      // NULL, or fp32 [2D]: learnable gain of the output norm; then yg = y * gain is written too
  __half* yg;             // [B*H, N, 2D] dense (only with gain)
};

__device__ __forceinline__ float load_lambda(const void* p, int dtype) {
  if (dtype == 0) return __half2float(*reinterpret_cast<const __half*>(p));
  if (dtype == 2) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
  return *reinterpret_cast<const float*>(p);
}


namespace fwd64 {
constexpr int BM = 128;            // query rows per CTA
constexpr int BN = 128;            // key/value rows per shared-memory tile
constexpr int SUB = 64;            // key/value rows per MMA sub-tile (one S buffer in TMEM)
constexpr int HD = 64;
constexpr int DV = 128;
constexpr int KS = 3;              // K ring depth
constexpr int VS = 2;              // V ring depth
constexpr int Q_BYTES = BM * HD * 2;            // 16 KB per Q
constexpr int K_BYTES = BN * HD * 2;            // 16 KB per K
constexpr int V_BYTES = BN * DV * 2;            // 32 KB (two 64-column boxes)
constexpr int OFF_Q1 = 0;
constexpr int OFF_Q2 = Q_BYTES;
constexpr int OFF_K = 2 * Q_BYTES;                       // stage s: K1 at +s*2*K_BYTES, K2 right after
constexpr int OFF_V = OFF_K + KS * 2 * K_BYTES;
constexpr int OFF_MISC = OFF_V + VS * V_BYTES;           // barriers, coefficients
constexpr int PRELOAD = 2;                               // key/value tiles requested before the setup barrier (<= KS, VS)
constexpr int STORE_TILE_BYTES = BM * 128;               // epilogue staging: 128 rows x 64 columns x 2 bytes
static_assert(6 * STORE_TILE_BYTES <= KS * 2 * K_BYTES, "the y / a2 / gained-y staging tiles reuse the K ring");
// TMEM columns: S_b buffer u at 128*b + 64*u; O1 at 256, O2 at 384
constexpr int T_O = 256;

}  // namespace fwd64

__device__ __forceinline__ float max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

}  // namespace da
