// C ABI of libdiffattn (see include/diffattn.h): argument checks, TMA descriptors, launches.
// Single translation unit: the kernels live in the .cuh files included below.
#include "../../include/diffattn.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "bwd.cuh"
#include "bwd128.cuh"
#include "bwd_fused64.cuh"
#include "fwd.cuh"
#include "fwd64.cuh"
#include "fwd128.cuh"
#include "sm100.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define DA_CUDA(call)                                                                       \
  do {                                                                                      \
    cudaError_t e_ = (call);                                                                \
    if (e_ != cudaSuccess) return fail(DIFFATTN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

constexpr int kMaxDevices = 64;

// Makes `device` current for the lifetime of the object and puts the caller's device back afterwards.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  int enter(int device) {
    if (device < 0 || device >= kMaxDevices) return fail(DIFFATTN_ERR_BAD_SHAPE, "device ordinal %d outside [0,%d)", device, kMaxDevices);
    DA_CUDA(cudaGetDevice(&prev));
    if (prev != device) {
      DA_CUDA(cudaSetDevice(device));
      switched = true;
    }
    return DIFFATTN_OK;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// ---- host-side caches, one set per calling thread (no lock, no shared mutable state): encoded tensor maps, launch
// attributes already set, SM counts, and the device every base pointer was found on.  A tensor map is a pure
// function of its key, so an entry never goes stale; the pointer cache keeps only pointers that passed (a pointer
// freed and handed out again by another device's allocator would be re-checked only after the cache was flushed:
// caches are flushed when they grow past kCacheLimit entries).  Measured at B2 H4 N128 (host clock around 1000
// enqueues): the caches save nothing -- encoding a map costs about as much as finding one -- and a call costs
// what its three or four launches cost; they are kept for the device check, which would otherwise query the
// driver for every pointer of every call.
struct MapKey {
  const void* base;
  int64_t s_row, s2, s3;
  int32_t cols, rows, d2, d3, box_rows, bf;
  bool operator==(const MapKey& o) const {
    return base == o.base && s_row == o.s_row && s2 == o.s2 && s3 == o.s3 && cols == o.cols && rows == o.rows && d2 == o.d2 &&
           d3 == o.d3 && box_rows == o.box_rows && bf == o.bf;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    auto mix = [&](uint64_t v) { h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); };
    mix(uint64_t(k.s_row)); mix(uint64_t(k.s2)); mix(uint64_t(k.s3));
    mix((uint64_t(uint32_t(k.cols)) << 32) | uint32_t(k.rows));
    mix((uint64_t(uint32_t(k.d2)) << 32) | uint32_t(k.d3));
    mix((uint64_t(uint32_t(k.box_rows)) << 1) | uint32_t(k.bf));
    return size_t(h);
  }
};
constexpr size_t kCacheLimit = 4096;
thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
thread_local std::unordered_map<const void*, uint64_t> g_attr_done;     // kernel -> bit per device: dynamic shared memory size set
thread_local std::unordered_map<const void*, int> g_ptr_device;         // base pointer -> device ordinal it was verified on
thread_local int g_sm_count[kMaxDevices] = {0};

// 16-bit (fp16, or bf16 when BF) tensor [d3, d2, rows, cols] with element strides (s3, s2, s_row, 1); box = box_rows x 64 columns,
// 128-byte swizzle (the layout the tcgen05 shared-memory descriptors in sm100.cuh describe).
template <bool BF>
int make_map(CUtensorMap* map, const void* base, int cols, int rows, int d2, int d3, int64_t s_row, int64_t s2, int64_t s3,
             int box_rows, const char* what) {
  const MapKey key{base, s_row, s2, s3, cols, rows, d2, d3, box_rows, BF ? 1 : 0};
  {
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *map = it->second;
      return DIFFATTN_OK;
    }
  }
  auto enc = get_encode();
  if (!enc) return fail(DIFFATTN_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[4] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(d2), cuuint64_t(d3)};
  cuuint64_t strides[3] = {cuuint64_t(s_row) * 2, cuuint64_t(s2) * 2, cuuint64_t(s3) * 2};
  // a size-1 dimension's stride is never used, but the encoder still wants a legal value
  if (d2 == 1) strides[1] = strides[0] * cuuint64_t(rows);
  if (d3 == 1) strides[2] = strides[1] * cuuint64_t(d2);
  // The box is always 64 columns (128 bytes, one swizzle row).  A tensor narrower than that (head dim 32)
  // is padded by the TMA engine: out-of-range elements arrive as zeros.
  cuuint32_t box[4] = {64, cuuint32_t(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = enc(map, BF ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DIFFATTN_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, int(r));
  if (g_maps.size() >= kCacheLimit) g_maps.clear();
  g_maps.emplace(key, *map);
  return DIFFATTN_OK;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize, once per kernel and device
template <typename K>
int set_smem(K kernel, int bytes, int device) {
  const void* key = reinterpret_cast<const void*>(kernel);
  auto it = g_attr_done.find(key);
  if (it != g_attr_done.end() && ((it->second >> device) & 1ull)) return DIFFATTN_OK;
  DA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  g_attr_done[key] |= 1ull << device;
  return DIFFATTN_OK;
}

int sm_count(int device) {
  if (g_sm_count[device] > 0) return g_sm_count[device];
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
  g_sm_count[device] = sms;
  return sms;
}

// Every tensor must be device (or managed) memory of `device`: a host pointer or another GPU's buffer would make
// the kernels fault.  Looked up once per new base pointer.
int check_on_device(const void* ptr, int device, const char* what) {
  if (!ptr) return DIFFATTN_OK;
  {
    auto it = g_ptr_device.find(ptr);
    if (it != g_ptr_device.end() && it->second == device) return DIFFATTN_OK;
  }
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(DIFFATTN_ERR_CUDA, "cudaPointerGetAttributes(%s): %s", what, cudaGetErrorString(e));
  }
  if (attr.type == cudaMemoryTypeManaged) return DIFFATTN_OK;
  if (attr.type != cudaMemoryTypeDevice)
    return fail(DIFFATTN_ERR_WRONG_DEVICE, "%s (%p) is not device memory (host or unregistered pointer)", what, ptr);
  if (attr.device != device)
    return fail(DIFFATTN_ERR_WRONG_DEVICE, "%s (%p) lives on device %d but the call names device %d", what, ptr, attr.device, device);
  if (g_ptr_device.size() >= kCacheLimit) g_ptr_device.clear();
  g_ptr_device[ptr] = device;
  return DIFFATTN_OK;
}

int check_pointers_on_device(const DiffAttnParams* p, bool bwd) {
  int rc;
  const void* fp[] = {p->q1, p->q2, p->k1, p->k2, p->v, p->lambda_scale, p->y, p->a2, p->lse1, p->lse2, p->rstd, p->gain, p->y_gained};
  const char* fn[] = {"q1", "q2", "k1", "k2", "v", "lambda_scale", "y", "a2", "lse1", "lse2", "rstd", "gain", "y_gained"};
  for (int i = 0; i < 13; ++i)
    if ((rc = check_on_device(fp[i], p->device, fn[i]))) return rc;
  if (bwd) {
    const void* bp[] = {p->dy, p->dq1, p->dq2, p->dk1, p->dk2, p->dv, p->dlambda, p->workspace, p->dgain};
    const char* bn[] = {"dy", "dq1", "dq2", "dk1", "dk2", "dv", "dlambda", "workspace", "dgain"};
    for (int i = 0; i < 9; ++i)
      if ((rc = check_on_device(bp[i], p->device, bn[i]))) return rc;
  }
  return DIFFATTN_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// the single-pass backward (bwd_fused64.cuh) exists for head dims 32 and 64 and is opt-in
bool fused_form(const DiffAttnParams* p) { return p->single_pass && p->D <= 64; }

int check_common(const DiffAttnParams* p, bool bwd) {
  if (!p) return fail(DIFFATTN_ERR_NULL_PTR, "params is NULL");
  if (p->struct_size != sizeof(DiffAttnParams))
    return fail(DIFFATTN_ERR_BAD_STRUCT, "struct_size %u != %zu", p->struct_size, sizeof(DiffAttnParams));
  if (p->B < 0 || p->H < 0 || p->N < 0 || p->D <= 0)
    return fail(DIFFATTN_ERR_BAD_SHAPE, "negative size: B=%d H=%d N=%d D=%d", p->B, p->H, p->N, p->D);
  if (!diffattn_supports(p->D, bwd ? 1 : 0))
    return fail(DIFFATTN_ERR_UNSUPPORTED_D, "head dim %d is not compiled in (supported: 32, 64, 128)", p->D);
  if (p->lambda_dtype != DIFFATTN_LAMBDA_F16 && p->lambda_dtype != DIFFATTN_LAMBDA_F32 && p->lambda_dtype != DIFFATTN_LAMBDA_BF16)
    return fail(DIFFATTN_ERR_BAD_DTYPE, "lambda_dtype %d unknown", p->lambda_dtype);
  if (p->io_dtype != DIFFATTN_IO_F16 && p->io_dtype != DIFFATTN_IO_BF16)
    return fail(DIFFATTN_ERR_BAD_DTYPE, "io_dtype %d unknown", p->io_dtype);
  if (p->gain && (!p->y_gained || !aligned16(p->gain) || !aligned16(p->y_gained)))
    return fail(p->y_gained ? DIFFATTN_ERR_MISALIGNED : DIFFATTN_ERR_NULL_PTR, "gain given: y_gained must be set, both 16-byte aligned");
  if (p->gain && bwd && !p->dgain) return fail(DIFFATTN_ERR_NULL_PTR, "gain given: dgain is NULL");
  if (p->dropout_threshold > 255)
    return fail(DIFFATTN_ERR_BAD_SHAPE, "dropout_threshold %u exceeds 255", p->dropout_threshold);
  if (p->dropout_threshold && p->N > 131072)      // the mask's counter packs (row >> 1, column >> 1) into 16 + 16 bits
    return fail(DIFFATTN_ERR_BAD_SHAPE, "dropout supports N <= 131072 (got %d)", p->N);
  if ((long long)p->B * p->H > 65535)
    return fail(DIFFATTN_ERR_BAD_SHAPE, "B*H=%lld exceeds the grid limit 65535", (long long)p->B * p->H);
  if (p->B == 0 || p->H == 0 || p->N == 0) return 1;   // empty: nothing to do
  const void* ptrs[] = {p->q1, p->q2, p->k1, p->k2, p->v, p->lambda_scale, p->y, p->a2, p->lse1, p->lse2, p->rstd};
  const char* names[] = {"q1", "q2", "k1", "k2", "v", "lambda_scale", "y", "a2", "lse1", "lse2", "rstd"};
  for (int i = 0; i < 11; ++i)
    if (!ptrs[i]) return fail(DIFFATTN_ERR_NULL_PTR, "%s is NULL", names[i]);
  for (int i = 0; i < 5; ++i)
    if (!aligned16(ptrs[i])) return fail(DIFFATTN_ERR_MISALIGNED, "%s is not 16-byte aligned", names[i]);
  if (!aligned16(p->y) || !aligned16(p->a2)) return fail(DIFFATTN_ERR_MISALIGNED, "y/a2 not 16-byte aligned");
  const int64_t st[] = {p->qk_stride_b, p->qk_stride_h, p->qk_stride_n, p->v_stride_b, p->v_stride_h, p->v_stride_n};
  for (int i = 0; i < 6; ++i)
    if (st[i] <= 0 || st[i] % 8 != 0)
      return fail(DIFFATTN_ERR_BAD_STRIDE, "stride %d = %lld must be a positive multiple of 8 elements", i, (long long)st[i]);
  if (p->qk_stride_n < p->D || p->v_stride_n < 2 * p->D)
    return fail(DIFFATTN_ERR_BAD_STRIDE, "row stride smaller than the row");
  if (bwd) {
    const void* bp[] = {p->dy, p->dq1, p->dq2, p->dk1, p->dk2, p->dv, p->dlambda};
    const char* bn[] = {"dy", "dq1", "dq2", "dk1", "dk2", "dv", "dlambda"};
    for (int i = 0; i < 7; ++i)
      if (!bp[i]) return fail(DIFFATTN_ERR_NULL_PTR, "%s is NULL", bn[i]);
    for (int i = 0; i < 6; ++i)
      if (!aligned16(bp[i])) return fail(DIFFATTN_ERR_MISALIGNED, "%s is not 16-byte aligned", bn[i]);
    const uint64_t need = diffattn_workspace_bytes(p);
    if (!p->workspace || p->workspace_bytes < need)
      return fail(DIFFATTN_ERR_WORKSPACE, "workspace %llu bytes, need %llu", (unsigned long long)p->workspace_bytes,
                  (unsigned long long)need);
    if (reinterpret_cast<uintptr_t>(p->workspace) & 255) return fail(DIFFATTN_ERR_MISALIGNED, "workspace not 256-byte aligned");
  }
  return DIFFATTN_OK;
}

uint64_t round256(uint64_t x) { return (x + 255) & ~uint64_t(255); }

}  // namespace

extern "C" {

const char* diffattn_last_error(void) { return g_err; }
int diffattn_version(void) { return DIFFATTN_VERSION; }
// the same head dims are compiled in for both directions
int diffattn_supports(int32_t d, int32_t dir) {
  if (dir != 0 && dir != 1) return 0;
  return (d == 64 || d == 32 || d == 128) ? 1 : 0;
}

uint64_t diffattn_workspace_bytes(const DiffAttnParams* p) {
  if (!p || p->B <= 0 || p->H <= 0 || p->N <= 0 || p->D <= 0) return 0;
  const uint64_t rows = uint64_t(p->B) * p->H * p->N;
  const uint64_t n_pad = (uint64_t(p->N) + 127) & ~uint64_t(127);
  // dA fp16 [B*H, N, 2D] + per-row statistics {lse1', lse2', E1, E2} with a row pitch of N rounded up to 128
  uint64_t bytes = round256(rows * 2 * p->D * 2) + round256(uint64_t(p->B) * p->H * n_pad * 16);
  // single-pass form: fp32 partial sums of dQ1, dQ2, [2][B*H][n_pad][64]
  if (fused_form(p)) bytes += round256(2 * uint64_t(p->B) * p->H * n_pad * 64 * 4);
  return bytes;
}

}  // extern "C"

namespace {

template <bool BF, bool DROP>
int fwd_impl(const DiffAttnParams* p) {
  int rc = 0;
  DeviceGuard guard;
  if ((rc = guard.enter(p->device))) return rc;
  if ((rc = check_pointers_on_device(p, false))) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  CUtensorMap mq1, mq2, mk1, mk2, mv;
  const int D = p->D, DV = 2 * p->D;
  const int kv_rows = D == 128 ? 64 : 128;      // the D = 128 kernel streams 64-row tiles
  if ((rc = make_map<BF>(&mq1, p->q1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "q1"))) return rc;
  if ((rc = make_map<BF>(&mq2, p->q2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "q2"))) return rc;
  if ((rc = make_map<BF>(&mk1, p->k1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, kv_rows, "k1"))) return rc;
  if ((rc = make_map<BF>(&mk2, p->k2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, kv_rows, "k2"))) return rc;
  if ((rc = make_map<BF>(&mv, p->v, DV, p->N, p->H, p->B, p->v_stride_n, p->v_stride_h, p->v_stride_b, kv_rows, "v"))) return rc;
  da::FwdArgs a;
  a.y = static_cast<__half*>(p->y);
  a.a2 = static_cast<__half*>(p->a2);
  a.lse1 = p->lse1; a.lse2 = p->lse2; a.rstd = p->rstd;
  a.lambda_ptr = p->lambda_scale; a.lambda_dtype = p->lambda_dtype;
  a.sm_scale = p->sm_scale; a.out_scale = 1.f - p->lambda_init; a.eps = p->eps;
  a.rms_norm = p->rms_norm; a.n = p->N; a.h = p->H; a.d = p->D; a.causal = p->causal ? 1 : 0;
  a.drop_thresh = p->dropout_threshold; a.seed_lo = uint32_t(p->dropout_seed); a.seed_hi = uint32_t(p->dropout_seed >> 32);
  a.drop_scale = 256.f / float(256u - p->dropout_threshold);
  a.gain = p->gain; a.yg = static_cast<__half*>(p->y_gained);
  if (D == 128) {
    // one CTA per branch; the two CTAs of a query tile form a cluster and exchange A2 through distributed shared memory
    if ((rc = set_smem(da::diffattn_fwd128_branch_kernel<BF, DROP>, da::fwd128::SMEM_BYTES, p->device))) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p->N + 127) / 128, p->B * p->H, 2);
    cfg.blockDim = dim3(da::fwd128::NUM_THREADS);
    cfg.dynamicSmemBytes = da::fwd128::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 2;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DA_CUDA(cudaLaunchKernelEx(&cfg, da::diffattn_fwd128_branch_kernel<BF, DROP>, mq1, mq2, mk1, mk2, mv, a));
    return DIFFATTN_OK;
  }
  // outputs leave through TMA stores: dense [B*H, N, 2D] maps with 128-row boxes
  CUtensorMap my, ma2;
  const long long bh = (long long)p->B * p->H;
  if ((rc = make_map<BF>(&my, p->y, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 128, "y"))) return rc;
  if ((rc = make_map<BF>(&ma2, p->a2, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 128, "a2"))) return rc;
  CUtensorMap myg = my;      // only read by the kernel when a gain is given
  if (p->gain && (rc = make_map<BF>(&myg, p->y_gained, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 128, "y_gained"))) return rc;
  dim3 grid((p->N + 127) / 128, p->B * p->H);
  if ((rc = set_smem(da::diffattn_fwd64_kernel<BF, DROP>, da::fwd64::SMEM_BYTES, p->device))) return rc;
  da::diffattn_fwd64_kernel<BF, DROP><<<grid, da::fwd64::NUM_THREADS, da::fwd64::SMEM_BYTES, stream>>>(mq1, mq2, mk1, mk2, mv, my, ma2, myg, a);
  DA_CUDA(cudaGetLastError());
  return DIFFATTN_OK;
}

template <bool BF, bool DROP>
int bwd_impl(const DiffAttnParams* p, int32_t stages) {
  int rc = 0;
  DeviceGuard guard;
  if ((rc = guard.enter(p->device))) return rc;
  if ((rc = check_pointers_on_device(p, true))) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const int D = p->D, DV = 2 * p->D;
  const long long bh = (long long)p->B * p->H;
  const uint64_t rows = uint64_t(bh) * p->N;
  const bool fused = fused_form(p);
  da::BwdArgs a;
  a.y = static_cast<const __half*>(p->y);
  a.a2 = static_cast<const __half*>(p->a2);
  a.dy = static_cast<const __half*>(p->dy);
  a.lse1 = p->lse1; a.lse2 = p->lse2; a.rstd = p->rstd;
  a.n = p->N; a.h = p->H; a.d = p->D; a.rows = (long long)rows;
  a.n_pad = (p->N + 127) & ~127;
  uint8_t* ws = static_cast<uint8_t*>(p->workspace);
  a.da = reinterpret_cast<__half*>(ws);
  ws += round256(rows * DV * 2);
  a.stats = reinterpret_cast<float4*>(ws);
  ws += round256(uint64_t(bh) * a.n_pad * 16);
  a.dq_acc = fused ? reinterpret_cast<float*>(ws) : nullptr;
  a.dq_acc_f4 = fused ? (long long)(2 * uint64_t(bh) * a.n_pad * 64 / 4) : 0;
  a.dq1 = static_cast<__half*>(p->dq1); a.dq2 = static_cast<__half*>(p->dq2);
  a.dk1 = static_cast<__half*>(p->dk1); a.dk2 = static_cast<__half*>(p->dk2);
  a.dv = static_cast<__half*>(p->dv);
  a.dlambda = p->dlambda;
  a.lambda_ptr = p->lambda_scale; a.lambda_dtype = p->lambda_dtype;
  a.sm_scale = p->sm_scale; a.out_scale = 1.f - p->lambda_init; a.rms_norm = p->rms_norm;
  a.causal = p->causal ? 1 : 0;
  a.drop_thresh = p->dropout_threshold; a.seed_lo = uint32_t(p->dropout_seed); a.seed_hi = uint32_t(p->dropout_seed >> 32);
  a.drop_scale = 256.f / float(256u - p->dropout_threshold);
  a.gain = p->gain; a.dgain = p->dgain;
  const int n_tiles = a.n_pad / 128;
  const int sms = sm_count(p->device);

  // 1. preprocess (grid-stride; one atomic per CTA for d(lambda)); zeroes the dQ partial sums of the single-pass form
  if (stages & DIFFATTN_STAGE_PRE) {
    long long blocks = (long long)((rows + 7) / 8);
    if (blocks > (long long)sms * 8) blocks = (long long)sms * 8;
    if (D == 128) da::diffattn_bwd_pre_kernel<8, BF><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (D == 64) da::diffattn_bwd_pre_kernel<4, BF><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else da::diffattn_bwd_pre_kernel<2, BF><<<(unsigned)blocks, 256, 0, stream>>>(a);
    if (a.n_pad != a.n) da::diffattn_bwd_padstats_kernel<<<64, 256, 0, stream>>>(a, (int)bh);
    DA_CUDA(cudaGetLastError());
  }
  if (D == 128) {
    // D = 128: dV kernel, then dK and dQ through the per-branch "side" kernel (bwd128.cuh)
    auto qk = [&](CUtensorMap* m, const void* ptr, int box_rows, const char* nm) {
      return make_map<BF>(m, ptr, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, box_rows, nm);
    };
    CUtensorMap q1_64, q2_64, k1_64, k2_64, q1_128, q2_128, k1_128, k2_128, v_64, v_128, da_64, da_128;
    if (stages & DIFFATTN_STAGE_DKDV) {
      if ((rc = qk(&q1_64, p->q1, 64, "q1"))) return rc;
      if ((rc = qk(&q2_64, p->q2, 64, "q2"))) return rc;
      if ((rc = qk(&k1_128, p->k1, 128, "k1"))) return rc;
      if ((rc = qk(&k2_128, p->k2, 128, "k2"))) return rc;
      if ((rc = make_map<BF>(&v_128, p->v, DV, p->N, p->H, p->B, p->v_stride_n, p->v_stride_h, p->v_stride_b, 128, "v"))) return rc;
      if ((rc = make_map<BF>(&da_64, a.da, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 64, "dA"))) return rc;
      if ((rc = set_smem(da::diffattn_bwd_dv128_kernel<BF, DROP>, da::dv128::SMEM_BYTES, p->device))) return rc;
      dim3 g1(n_tiles, (unsigned)bh);
      da::diffattn_bwd_dv128_kernel<BF, DROP><<<g1, da::dv128::NUM_THREADS, da::dv128::SMEM_BYTES, stream>>>(q1_64, q2_64, k1_128, k2_128, da_64, a);
      DA_CUDA(cudaGetLastError());
      if ((rc = set_smem(da::diffattn_bwd_side128_kernel<false, BF, DROP>, da::side128::SMEM_BYTES, p->device))) return rc;
      dim3 g2(n_tiles, (unsigned)bh, 2);
      da::diffattn_bwd_side128_kernel<false, BF, DROP><<<g2, da::side128::NUM_THREADS, da::side128::SMEM_BYTES, stream>>>(
          k1_128, k2_128, v_128, q1_64, q2_64, da_64, a);
      DA_CUDA(cudaGetLastError());
    }
    if (stages & DIFFATTN_STAGE_DQ) {
      if ((rc = qk(&q1_128, p->q1, 128, "q1"))) return rc;
      if ((rc = qk(&q2_128, p->q2, 128, "q2"))) return rc;
      if ((rc = qk(&k1_64, p->k1, 64, "k1"))) return rc;
      if ((rc = qk(&k2_64, p->k2, 64, "k2"))) return rc;
      if ((rc = make_map<BF>(&v_64, p->v, DV, p->N, p->H, p->B, p->v_stride_n, p->v_stride_h, p->v_stride_b, 64, "v"))) return rc;
      if ((rc = make_map<BF>(&da_128, a.da, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 128, "dA"))) return rc;
      if ((rc = set_smem(da::diffattn_bwd_side128_kernel<true, BF, DROP>, da::side128::SMEM_BYTES, p->device))) return rc;
      dim3 g3(n_tiles, (unsigned)bh, 2);
      da::diffattn_bwd_side128_kernel<true, BF, DROP><<<g3, da::side128::NUM_THREADS, da::side128::SMEM_BYTES, stream>>>(
          q1_128, q2_128, da_128, k1_64, k2_64, v_64, a);
      DA_CUDA(cudaGetLastError());
    }
    return DIFFATTN_OK;
  }
  CUtensorMap mq1, mq2, mk1, mk2, mv, mda;
  if (stages & (DIFFATTN_STAGE_DKDV | DIFFATTN_STAGE_FUSED)) {
    // key/value tiles of 128 rows resident, query-side tiles of 64 rows streamed
    if ((rc = make_map<BF>(&mq1, p->q1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 64, "q1"))) return rc;
    if ((rc = make_map<BF>(&mq2, p->q2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 64, "q2"))) return rc;
    if ((rc = make_map<BF>(&mk1, p->k1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "k1"))) return rc;
    if ((rc = make_map<BF>(&mk2, p->k2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "k2"))) return rc;
    if ((rc = make_map<BF>(&mv, p->v, DV, p->N, p->H, p->B, p->v_stride_n, p->v_stride_h, p->v_stride_b, 128, "v"))) return rc;
    if ((rc = make_map<BF>(&mda, a.da, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 64, "dA"))) return rc;
    // gradients leave through TMA stores: dense [B*H, N, D] / [B*H, N, 2D] maps with 128-row boxes
    CUtensorMap mdk1, mdk2, mdv;
    auto grad_map = [&](CUtensorMap* m, void* ptr, int cols, const char* nm) {
      return make_map<BF>(m, ptr, cols, p->N, (int)bh, 1, cols, (int64_t)p->N * cols, (int64_t)p->N * cols * bh, 128, nm);
    };
    if ((rc = grad_map(&mdk1, p->dk1, D, "dk1"))) return rc;
    if ((rc = grad_map(&mdk2, p->dk2, D, "dk2"))) return rc;
    if ((rc = grad_map(&mdv, p->dv, DV, "dv"))) return rc;
    dim3 grid(n_tiles, (unsigned)bh);
    if (stages & DIFFATTN_STAGE_FUSED) {
      // 2. single pass: dK1, dK2, dV and the partial sums of dQ1, dQ2
      if ((rc = set_smem(da::diffattn_bwd_fused64_kernel<BF, DROP>, da::fused64::SMEM_BYTES, p->device))) return rc;
      da::diffattn_bwd_fused64_kernel<BF, DROP><<<grid, da::fused64::NUM_THREADS, da::fused64::SMEM_BYTES, stream>>>(mq1, mq2, mk1, mk2, mv, mda, mdk1, mdk2, mdv, a);
    } else {
      // 2'. dK, dV only (two-kernel form)
      if ((rc = set_smem(da::diffattn_bwd_dkdv64_kernel<BF, DROP>, da::dkdv64::SMEM_BYTES, p->device))) return rc;
      da::diffattn_bwd_dkdv64_kernel<BF, DROP><<<grid, da::dkdv64::NUM_THREADS, da::dkdv64::SMEM_BYTES, stream>>>(mq1, mq2, mk1, mk2, mv, mda, mdk1, mdk2, mdv, a);
    }
    DA_CUDA(cudaGetLastError());
  }
  if (stages & DIFFATTN_STAGE_DQ_FINISH) {
    // 3. dQ = sm_scale * partial sums, converted to the 16-bit type
    long long blocks = (long long)((2 * rows * (D / 8) + 255) / 256);
    if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
    da::diffattn_bwd_dq_finish_kernel<BF><<<(unsigned)blocks, 256, 0, stream>>>(a, (int)bh);
    DA_CUDA(cudaGetLastError());
  }
  if (stages & DIFFATTN_STAGE_DQ) {
    // 3'. dQ (two-kernel form): query tiles of 128 rows resident, key/value tiles of 128 rows streamed
    if ((rc = make_map<BF>(&mq1, p->q1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "q1"))) return rc;
    if ((rc = make_map<BF>(&mq2, p->q2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "q2"))) return rc;
    if ((rc = make_map<BF>(&mk1, p->k1, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "k1"))) return rc;
    if ((rc = make_map<BF>(&mk2, p->k2, D, p->N, p->H, p->B, p->qk_stride_n, p->qk_stride_h, p->qk_stride_b, 128, "k2"))) return rc;
    if ((rc = make_map<BF>(&mv, p->v, DV, p->N, p->H, p->B, p->v_stride_n, p->v_stride_h, p->v_stride_b, 128, "v"))) return rc;
    if ((rc = make_map<BF>(&mda, a.da, DV, p->N, (int)bh, 1, DV, (int64_t)p->N * DV, (int64_t)p->N * DV * bh, 128, "dA"))) return rc;
    if ((rc = set_smem(da::diffattn_bwd_dq64_kernel<BF, DROP>, da::dq64::SMEM_BYTES, p->device))) return rc;
    dim3 grid(n_tiles, (unsigned)bh);
    da::diffattn_bwd_dq64_kernel<BF, DROP><<<grid, da::dq64::NUM_THREADS, da::dq64::SMEM_BYTES, stream>>>(mq1, mq2, mk1, mk2, mv, mda, a);
    DA_CUDA(cudaGetLastError());
  }
  return DIFFATTN_OK;
}

int all_stages(const DiffAttnParams* p) {
  return fused_form(p) ? (DIFFATTN_STAGE_PRE | DIFFATTN_STAGE_FUSED | DIFFATTN_STAGE_DQ_FINISH)
                       : (DIFFATTN_STAGE_PRE | DIFFATTN_STAGE_DKDV | DIFFATTN_STAGE_DQ);
}

}  // namespace

extern "C" {

int diffattn_fwd(const DiffAttnParams* p) {
  const int rc = check_common(p, false);
  if (rc < 0) return rc;
  if (rc == 1) return DIFFATTN_OK;
  const bool bf = p->io_dtype == DIFFATTN_IO_BF16;
#ifdef DA_MINIMAL_BUILD      // tuning builds: fp16 without dropout only (a quarter of the compile time)
  if (bf || p->dropout_threshold) return fail(DIFFATTN_ERR_BAD_DTYPE, "this build holds the fp16, no-dropout kernels only");
  return fwd_impl<false, false>(p);
#else
  if (p->dropout_threshold) return bf ? fwd_impl<true, true>(p) : fwd_impl<false, true>(p);
  return bf ? fwd_impl<true, false>(p) : fwd_impl<false, false>(p);
#endif
}

int diffattn_bwd(const DiffAttnParams* p) {
  if (!p) return fail(DIFFATTN_ERR_NULL_PTR, "params is NULL");
  if (p->struct_size != sizeof(DiffAttnParams))
    return fail(DIFFATTN_ERR_BAD_STRUCT, "struct_size %u != %zu", p->struct_size, sizeof(DiffAttnParams));
  return diffattn_bwd_stages(p, all_stages(p));
}

int diffattn_bwd_stages(const DiffAttnParams* p, int32_t stages) {
  const int rc = check_common(p, true);
  if (rc < 0) return rc;
  if (rc == 1) return DIFFATTN_OK;
  if (stages & ~all_stages(p))
    return fail(DIFFATTN_ERR_BAD_SHAPE, "stages 0x%x: this call's form (single_pass=%d, D=%d) has stages 0x%x only", stages,
                p->single_pass, p->D, all_stages(p));
  const bool bf = p->io_dtype == DIFFATTN_IO_BF16;
#ifdef DA_MINIMAL_BUILD
  if (bf || p->dropout_threshold) return fail(DIFFATTN_ERR_BAD_DTYPE, "this build holds the fp16, no-dropout kernels only");
  return bwd_impl<false, false>(p, stages);
#else
  if (p->dropout_threshold) return bf ? bwd_impl<true, true>(p, stages) : bwd_impl<false, true>(p, stages);
  return bf ? bwd_impl<true, false>(p, stages) : bwd_impl<false, false>(p, stages);
#endif
}

// ---- allocation-free backward: scratch in a file-scope device array -------------------------------
// In host code the array's name is only a handle for the runtime, not a device address; the address
// each device gives it is looked up once per device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) unsigned char g_static_scratch[DIFFATTN_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};
}  // namespace

int diffattn_bwd_static(const DiffAttnParams* p) {
  if (!p) return fail(DIFFATTN_ERR_NULL_PTR, "params is NULL");
  if (p->struct_size != sizeof(DiffAttnParams))
    return fail(DIFFATTN_ERR_BAD_STRUCT, "struct_size %u != %zu", p->struct_size, sizeof(DiffAttnParams));
  const uint64_t need = diffattn_workspace_bytes(p);
  if (need == 0) {
    // empty or malformed shape: the ordinary checks decide (an empty shape is OK), without touching the device
    DiffAttnParams q = *p;
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    return diffattn_bwd_stages(&q, all_stages(&q));
  }
  if (need > DIFFATTN_STATIC_SCRATCH_BYTES)
    return fail(DIFFATTN_ERR_WORKSPACE,
                "diffattn_bwd_static: this shape needs %llu scratch bytes, the built-in array holds %u; "
                "use diffattn_bwd with a caller workspace",
                (unsigned long long)need, unsigned(DIFFATTN_STATIC_SCRATCH_BYTES));
  if (p->device < 0 || p->device >= kMaxDevices)
    return fail(DIFFATTN_ERR_BAD_SHAPE, "device ordinal %d outside [0,%d)", p->device, kMaxDevices);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[p->device]) {
      // set-up, once per device, with that device current
      DeviceGuard guard;
      int rc = guard.enter(p->device);
      if (rc) return rc;
      void* addr = nullptr;
      DA_CUDA(cudaGetSymbolAddress(&addr, g_static_scratch));
      if (!addr) return fail(DIFFATTN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
      g_static_ptr[p->device] = addr;
    }
    scratch = g_static_ptr[p->device];
  }
  DiffAttnParams q = *p;
  q.workspace = scratch;
  q.workspace_bytes = DIFFATTN_STATIC_SCRATCH_BYTES;
  return diffattn_bwd_stages(&q, all_stages(&q));
}

int diffattn_status(int32_t device) {
  DeviceGuard guard;
  int rc = guard.enter(device);
  if (rc) return rc;
  DA_CUDA(cudaDeviceSynchronize());
  int st[4] = {0, 0, 0, 0};
  DA_CUDA(cudaMemcpyFromSymbol(st, da::g_status, sizeof(st)));
  if (st[0] != 0) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(da::g_status, zero, sizeof(zero));
    return fail(DIFFATTN_ERR_TIMEOUT, "device-side wait gave up at site %d (block %d,%d iteration %d)", st[0], st[1], st[2], st[3]);
  }
  return DIFFATTN_OK;
}

}  // extern "C"
