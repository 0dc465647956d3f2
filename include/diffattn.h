/* C ABI of libdiffattn: differential attention forward/backward for NVIDIA B200 (sm_100a).
 *
 * This is the boundary the Python autograd function binds with ctypes.  It stands where the
 * reference's autograd Function launches its Triton kernels:
 *   diffattn_fwd  <->  _diff_attention.forward  (reference src/kernel.py:463-514, kernel :21-207)
 *   diffattn_bwd  <->  _diff_attention.backward (reference src/kernel.py:516-575, kernel :221-458)
 * The caller owns every buffer; the library never calls an allocator.  (Its image does carry one fixed
 * DIFFATTN_STATIC_SCRATCH_BYTES array per GPU, resident on every GPU that loads the library and used only
 * by diffattn_bwd_static.)  All device work is enqueued on `stream`; no call synchronises the host with the
 * device except diffattn_status().  Every entry point leaves the calling thread's current CUDA device as it
 * found it.  Every function returns 0 on success or a negative DIFFATTN_ERR_* code; nothing is launched
 * after a failed check.  diffattn_last_error() gives the message of the calling thread's last failure.
 * Host-side state: per calling thread, a cache of encoded TMA descriptors (keyed by base pointer, shape, strides,
 * box and type), of per-kernel launch attributes and of the device each base pointer was found on; nothing is
 * shared between threads except the address of the static scratch array (mutex).
 */
#ifndef DIFFATTN_H_
#define DIFFATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DIFFATTN_VERSION 2

enum {
  DIFFATTN_OK = 0,
  DIFFATTN_ERR_NULL_PTR = -1,
  DIFFATTN_ERR_BAD_STRUCT = -2,     /* struct_size does not match this library */
  DIFFATTN_ERR_BAD_SHAPE = -3,      /* negative sizes, B*H beyond the grid limit */
  DIFFATTN_ERR_UNSUPPORTED_D = -4,  /* head dim not compiled in */
  DIFFATTN_ERR_BAD_STRIDE = -5,     /* strides not a multiple of 8 elements (16 bytes) */
  DIFFATTN_ERR_MISALIGNED = -6,     /* base pointer not 16-byte aligned */
  DIFFATTN_ERR_BAD_DTYPE = -7,      /* lambda dtype tag unknown */
  DIFFATTN_ERR_WORKSPACE = -8,      /* workspace missing or too small */
  DIFFATTN_ERR_CUDA = -9,           /* a CUDA runtime/driver call failed */
  DIFFATTN_ERR_TIMEOUT = -10,       /* a device-side wait gave up (reported by diffattn_status) */
  DIFFATTN_ERR_WRONG_DEVICE = -11   /* a tensor pointer is not device memory of `device` (host memory, another GPU) */
};

enum { DIFFATTN_LAMBDA_F16 = 0, DIFFATTN_LAMBDA_F32 = 1, DIFFATTN_LAMBDA_BF16 = 2 };
/* 16-bit type of q1,q2,k1,k2,v,y,a2,dy and every gradient tensor.  The reference computes in fp16 only
 * (it casts P to tl.float16, src/kernel.py:175-176); bf16 is an extension for callers that train in bf16. */
enum { DIFFATTN_IO_F16 = 0, DIFFATTN_IO_BF16 = 1 };

/* ("fp16" below reads "bf16" when io_dtype = DIFFATTN_IO_BF16.)
 * q1,q2,k1,k2: fp16 [B,H,N,D] sharing one set of element strides (last dim contiguous), as the
 * reference takes them from Q1 alone (src/kernel.py:487-490).  v: fp16 [B,H,N,2D] with its own
 * strides (src/kernel.py:491-494).  Everything the library writes is dense row-major:
 * y, a2, dy, dv [B,H,N,2D] fp16; dq1,dq2,dk1,dk2 [B,H,N,D] fp16; lse1,lse2,rstd [B,H,N] fp32. */
typedef struct DiffAttnParams {
  uint32_t struct_size;            /* sizeof(DiffAttnParams) */
  int32_t device;                  /* CUDA device ordinal owning all pointers */
  void* stream;                    /* cudaStream_t */
  int32_t B, H, N, D;
  int64_t qk_stride_b, qk_stride_h, qk_stride_n;   /* in elements */
  int64_t v_stride_b, v_stride_h, v_stride_n;
  const void* q1; const void* q2; const void* k1; const void* k2; const void* v;
  const void* lambda_scale;        /* device pointer to ONE element (src/kernel.py:138,496) */
  int32_t lambda_dtype;            /* DIFFATTN_LAMBDA_* */
  int32_t rms_norm;                /* 0/1; (1 - lambda_init) is applied only when 1 (src/layers.py:74-78) */
  float sm_scale;                  /* 1/sqrt(D) (src/layers.py:20-22) */
  float lambda_init;
  float eps;                       /* 1e-5 (src/kernel.py:50) */
  int32_t causal;                  /* 0/1: 1 = key j is visible to query i only if j <= i (extension; the reference
                                      has no masking, README.md:2) */
  /* forward outputs (inputs of the backward) */
  void* y; void* a2; float* lse1; float* lse2; float* rstd;
  /* backward */
  const void* dy;
  void* dq1; void* dq2; void* dk1; void* dk2; void* dv;
  float* dlambda;                  /* ONE fp32 on the device; the backward ADDS -sum(E2) into it */
  void* workspace;                 /* diffattn_workspace_bytes() bytes, 256-byte aligned */
  uint64_t workspace_bytes;
  int32_t io_dtype;                /* DIFFATTN_IO_*: 0 = fp16 (the reference's type), 1 = bf16 */
  uint32_t dropout_threshold;      /* attention dropout (extension; the reference has none, README.md:2): 0 = off,
                                      else 1..255 = round(256 p): a probability is dropped when its hash byte is
                                      below the threshold, kept ones are scaled by 256/(256 - threshold).  The
                                      backward must be given the forward's threshold and seed.  N <= 131072 with dropout. */
  uint64_t dropout_seed;           /* the mask is a pure function of (seed, batch*head, branch, row, column) */
  /* Learnable gain of the output norm (extension: the reference's norm has no weight, src/layers.py:75; the layer it
   * adapts has one).  gain == NULL: off.  Otherwise gain is fp32 [2D] on the device; the forward writes y (without
   * the gain, kept for the backward) AND y_gained = y * gain (same type and shape as y, the layer's output); the
   * backward takes dy = d(loss)/d(y_gained) and ADDS sum over rows of dy * y into dgain (fp32 [2D]). */
  const float* gain;
  void* y_gained;
  float* dgain;
  /* Backward for head dims 32 and 64.  0 (default): two tensor-core kernels, the second of which recomputes the
   * scores per query block (as the reference's second loop does, src/kernel.py:426-436); every output tile has one
   * owner, the gradients are bit-reproducible.  1: ONE pass over the score tiles; every key block adds its share of
   * dQ1, dQ2 to an fp32 workspace with atomic adds, so dq1/dq2 can differ in the last bit between two runs (the
   * order of the adds is not fixed; dk1, dk2, dv are unaffected).  Measured on B200 the single pass is the slower
   * of the two (both forms move the same number of shared-memory bytes per score tile, which is what bounds them,
   * and the atomic adds come on top); it is kept as an option.  Ignored for head dim 128. */
  int32_t single_pass;
} DiffAttnParams;

/* Forward.  Reads q1,q2,k1,k2,v,lambda_scale; writes y,a2,lse1,lse2,rstd.
 * Replaces _diff_attention.forward + diff_attn_fwd (reference src/kernel.py:463-514, :21-207).
 * One kernel at every head dim; at head dim 128 its CTAs run in clusters of two (one per branch). */
int diffattn_fwd(const DiffAttnParams* p);

/* Backward.  Reads the forward's inputs and outputs plus dy; writes dq1,dq2,dk1,dk2,dv and adds the
 * lambda gradient into *dlambda (zero it first; partials of several shards add up on the host).
 * Replaces _diff_attention.backward + diff_attn_bwd (reference src/kernel.py:516-575, :221-458). */
int diffattn_bwd(const DiffAttnParams* p);

/* The backward is a few kernels; this entry runs a subset, for timing each kernel on its own.  Every later
 * stage reads what PRE wrote to the workspace (with single_pass = 1 PRE also zeroes the dQ partial sums).
 *   single_pass = 0 or head dim 128:  PRE, DKDV, DQ
 *   single_pass = 1, head dim <= 64:  PRE, FUSED (dK, dV and the dQ partial sums in one pass), DQ_FINISH
 * diffattn_bwd(p) runs the stages of p's form in that order; a stage that does not belong to p's form is
 * DIFFATTN_ERR_BAD_SHAPE.  (The reference's backward is one kernel, src/kernel.py:221-458: stage 1 at
 * :273-299, the dK/dV half at :410-424, the dQ half at :426-436.) */
enum { DIFFATTN_STAGE_PRE = 1, DIFFATTN_STAGE_DKDV = 2, DIFFATTN_STAGE_DQ = 4, DIFFATTN_STAGE_FUSED = 8,
       DIFFATTN_STAGE_DQ_FINISH = 16 };
int diffattn_bwd_stages(const DiffAttnParams* p, int32_t stages);

/* Backward without a caller-provided workspace and without any allocation.  (No counterpart in the
 * reference, whose backward allocates its scratch with torch on every call, src/kernel.py:520-529.)
 *
 * For whom: hosts that bind this ABI directly (C, ctypes, another runtime) and have no allocator to
 * hand: a serving loop that was given a fixed set of buffers up front, or a step loop that must not
 * call cudaMalloc because that call synchronises the whole device and can fail late under memory
 * pressure.  Such a caller passes inputs and outputs exactly as for diffattn_bwd and leaves
 * `workspace` / `workspace_bytes` unset (they are ignored).
 *
 * The scratch (dA and the per-row statistics) lives in one array of DIFFATTN_STATIC_SCRATCH_BYTES that
 * is part of the library image: every GPU that loads the library holds it until the process exits.
 * Limit: diffattn_workspace_bytes(p) must not exceed it (at D = 64: B*H*N <= 123361 rows; 42799 with
 * single_pass = 1), otherwise DIFFATTN_ERR_WORKSPACE is returned and nothing is launched.
 * The first call on each device looks the array's device address up (one cudaGetSymbolAddress, no
 * allocation) and keeps it; make that first call outside any stream capture.  The kept address is void
 * after cudaDeviceReset() of that device: do not reset a device between calls.  The call itself uses no
 * cudaMalloc, cudaFree or allocating library routine.  An empty shape (B, H or N = 0) returns 0 without
 * touching the device.
 * All calls on a device share the one array and it keeps what the previous call left there.  Nothing
 * in it has to start at zero (the preprocess kernel rewrites every byte the other kernels read), but
 * two calls whose kernels overlap on the GPU (different streams, no ordering) race on it: order
 * them.  *dlambda is still the caller's to zero. */
#define DIFFATTN_STATIC_SCRATCH_BYTES (32u << 20)
int diffattn_bwd_static(const DiffAttnParams* p);

/* Scratch bytes diffattn_bwd needs for these shapes and p->single_pass (the reference allocates its
 * D1/D2 and dLambda partial buffers itself, src/kernel.py:522-529).  The forward needs none. */
uint64_t diffattn_workspace_bytes(const DiffAttnParams* p);

/* Synchronises `device` and reads the device-side status word: 0, or DIFFATTN_ERR_TIMEOUT with the
 * site in diffattn_last_error().  Clears the word.  (No counterpart in the reference.) */
int diffattn_status(int32_t device);

const char* diffattn_last_error(void);   /* thread-local, never NULL */
int diffattn_version(void);
/* 1 when head dim d is compiled in for the forward (dir 0) / backward (dir 1) */
int diffattn_supports(int32_t d, int32_t dir);

#ifdef __cplusplus
}
#endif
#endif /* DIFFATTN_H_ */
