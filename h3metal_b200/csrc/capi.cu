// C ABI of libh3b200 (include/h3b200.h): context, error reporting, stream/timing/profiling, argument checks and
// TMA descriptor construction around the two kernels. Mirrors the conventions of the reference's Metal launcher
// (src/capi.mm of audenvenn/h3metal): thread-local error string, NULL / non-zero on failure, ordered asynchronous
// launches, a blocking wait that reports GPU time, and a per-launch profile mode.
#include "../../include/h3b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "kernels.h"

namespace {

thread_local std::string g_error;

int fail(const std::string &msg) {
  g_error = msg;
  return -1;
}
int fail_cuda(const char *what, cudaError_t e) {
  return fail(std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MapKey {
  const void *ptr;
  uint64_t dims[3], strides[2];  // extents (innermost first) and byte strides of dimensions 1 and 2
  uint32_t box[3];
  int rank, dtype, swizzle;
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && rank == o.rank && dtype == o.dtype && swizzle == o.swizzle &&
           memcmp(dims, o.dims, sizeof dims) == 0 && memcmp(strides, o.strides, sizeof strides) == 0 &&
           memcmp(box, o.box, sizeof box) == 0;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    for (uint64_t v : {k.dims[0], k.dims[1], k.dims[2], k.strides[0], k.strides[1], static_cast<uint64_t>(k.box[0]),
                       static_cast<uint64_t>(k.box[1]), static_cast<uint64_t>(k.box[2]), static_cast<uint64_t>(k.rank),
                       static_cast<uint64_t>(k.dtype), static_cast<uint64_t>(k.swizzle)})
      h = (h ^ v) * 0x100000001B3ull;
    return static_cast<size_t>(h);
  }
};

const char *status_text(int code) {
  switch (code) {
    case 1: return "TMA producer timed out waiting for a free shared-memory stage";
    case 2: return "MMA issuer timed out waiting for operands or a free accumulator";
    case 3: return "epilogue timed out waiting for an accumulator";
    case 4: return "wind-down timed out waiting for copies in flight";
    case 5: return "rotate+quantise kernel timed out waiting for a row to arrive in shared memory";
    case 6: return "self-test: the wait on a barrier nobody signals timed out";
    case 7: return "rendezvous of a row-parallel layer timed out: another GPU did not signal";
    default: return "unknown device status";
  }
}

}  // namespace

struct h3b_ctx {
  int device = 0;
  cudaDeviceProp prop{};
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_start = nullptr, ev_end = nullptr;
  bool timing_open = false;
  bool profile = false;
  std::vector<double> prof;
  int *status_dev = nullptr;   // device word the kernels write on a bounded-wait timeout
  int *status_host = nullptr;  // pinned copy read at wait
  EncodeTiledFn encode = nullptr;
  std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  int tile_n_override = 0, band_override = 0, pair_mode = 0, rot_threads = 0, rot_stages = 0, rot_chunk = 0;
  int overlap = 1;  // programmatic dependent launch of the path's main kernels (h3b_set_launch_overlap); on by default
  int pair_stages = 0, pair_clusters = 0;  // CTA-pair product: ring depth and resident clusters (0 = unavailable)
  int pair_stages_staged = 0;              // ring depth when 64 KB of shared memory stage the outputs for TMA stores
  int store_mode = 0;                      // staged (TMA) stores of the pair product: 0 automatic, 1 whenever possible, -1 never
  uint64_t launches = 0;
  std::string name;

  int make_current() {
    cudaError_t e = cudaSetDevice(device);
    return e == cudaSuccess ? 0 : fail_cuda("cudaSetDevice", e);
  }
  // Called before every launch: opens the timed region of the next wait.
  int before_launch(cudaEvent_t *prof_start) {
    if (make_current()) return -1;
    cudaError_t e;
    if (profile) {
      if ((e = cudaEventRecord(ev_start, stream)) != cudaSuccess) return fail_cuda("cudaEventRecord", e);
      *prof_start = ev_start;
    } else if (!timing_open) {
      if ((e = cudaEventRecord(ev_start, stream)) != cudaSuccess) return fail_cuda("cudaEventRecord", e);
      timing_open = true;
    }
    return 0;
  }
  int after_launch(const char *what, cudaError_t launch_err) {
    if (launch_err != cudaSuccess) return fail_cuda(what, launch_err);
    ++launches;
    if (profile) {
      cudaError_t e;
      if ((e = cudaEventRecord(ev_end, stream)) != cudaSuccess) return fail_cuda("cudaEventRecord", e);
      if ((e = cudaEventSynchronize(ev_end)) != cudaSuccess) return fail_cuda(what, e);
      float ms = 0;
      if ((e = cudaEventElapsedTime(&ms, ev_start, ev_end)) != cudaSuccess) return fail_cuda("cudaEventElapsedTime", e);
      prof.push_back(ms * 1e-3);
    }
    return 0;
  }
  // 2-D map of a row-major [rows][inner] tensor with a box of box_rows x box_inner elements.
  const CUtensorMap *tensor_map(const void *ptr, int dtype, uint64_t inner, uint64_t rows, uint64_t stride_bytes,
                                uint32_t box_inner, uint32_t box_rows, int swizzle) {
    MapKey key{};
    key.ptr = ptr; key.rank = 2; key.dtype = dtype; key.swizzle = swizzle;
    key.dims[0] = inner; key.dims[1] = rows; key.dims[2] = 1;
    key.strides[0] = stride_bytes; key.strides[1] = 0;
    key.box[0] = box_inner; key.box[1] = box_rows; key.box[2] = 1;
    return build_map(key);
  }
  // 3-D map {d0, d1, d2} (d0 innermost) with byte strides s1, s2 and a box {b0, b1, 1}.
  const CUtensorMap *tensor_map3(const void *ptr, int dtype, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                                 uint64_t s2, uint32_t b0, uint32_t b1, int swizzle) {
    MapKey key{};
    key.ptr = ptr; key.rank = 3; key.dtype = dtype; key.swizzle = swizzle;
    key.dims[0] = d0; key.dims[1] = d1; key.dims[2] = d2;
    key.strides[0] = s1; key.strides[1] = s2;
    key.box[0] = b0; key.box[1] = b1; key.box[2] = 1;
    return build_map(key);
  }
  const CUtensorMap *build_map(const MapKey &key) {
    auto it = maps.find(key);
    if (it != maps.end()) return &it->second;
    CUtensorMap m;
    if (encode_map(key, &m)) return nullptr;
    if (maps.size() > 4096) maps.clear();  // bound the cache; descriptors are cheap to rebuild
    return &maps.emplace(key, m).first->second;
  }
  // Encodes a descriptor into caller-provided storage (touches no cache, allocates nothing). 0 on success.
  int encode_map(const MapKey &key, CUtensorMap *out) {
    const cuuint64_t dims[3] = {key.dims[0], key.dims[1], key.dims[2]};
    const cuuint64_t strides[2] = {key.strides[0], key.strides[1]};
    const cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = key.dtype == h3b::kDtypeI8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : key.dtype == h3b::kDtypeBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : key.dtype == h3b::kDtypeF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = key.swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    const CUresult r = encode(out, dt, static_cast<cuuint32_t>(key.rank), const_cast<void *>(key.ptr), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      char buf[320];
      snprintf(buf, sizeof buf,
               "cuTensorMapEncodeTiled failed (%d) for ptr %p rank %d dims %llu x %llu x %llu strides %llu, %llu box %u x %u",
               (int)r, key.ptr, key.rank, (unsigned long long)dims[0], (unsigned long long)dims[1],
               (unsigned long long)dims[2], (unsigned long long)strides[0], (unsigned long long)strides[1], box[0], box[1]);
      return fail(buf);
    }
    return 0;
  }
  // 2-D descriptor either from the cache or, with cached == false, encoded into *local.
  const CUtensorMap *map2(bool cached, CUtensorMap *local, const void *ptr, int dtype, uint64_t inner, uint64_t rows,
                          uint64_t stride_bytes, uint32_t box_inner, uint32_t box_rows, int swizzle) {
    if (cached) return tensor_map(ptr, dtype, inner, rows, stride_bytes, box_inner, box_rows, swizzle);
    MapKey key{};
    key.ptr = ptr; key.rank = 2; key.dtype = dtype; key.swizzle = swizzle;
    key.dims[0] = inner; key.dims[1] = rows; key.dims[2] = 1;
    key.strides[0] = stride_bytes; key.strides[1] = 0;
    key.box[0] = box_inner; key.box[1] = box_rows; key.box[2] = 1;
    return encode_map(key, local) ? nullptr : local;
  }
};

// ---- scratch of the product with a LoRA term for callers that cannot allocate (h3b_gemm_w8a8_lora_noalloc) ----------
// Its T scratch lives in the library image instead of in caller memory: a file-scope device array. In host code the
// array's NAME is only a stand-in for the symbol, not a device address, so the address is fetched once per device
// with cudaGetSymbolAddress (below) and that pointer is what the kernels and the TMA descriptor receive.
static __device__ __align__(256) unsigned short g_lora_t_static[H3B_NOALLOC_MAX_T_VALUES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void *g_static_addr[kMaxDevices] = {};

// Device address of g_lora_t_static on `device`, which the caller has made current. Looked up once per device and
// remembered. h3b_open() calls this at set-up: the look-up makes the runtime load this file's device code, and with it
// place the array in that device's memory, while the context is allocating anyway - not in the middle of a caller's
// first no-alloc product.
void *static_scratch(int device) {
  if (device < 0 || device >= kMaxDevices) {
    fail("no-alloc product: device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_addr[device]) {
    void *ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_lora_t_static);
    if (e != cudaSuccess || !ptr) {
      fail_cuda("cudaGetSymbolAddress(static LoRA scratch)", e == cudaSuccess ? cudaErrorUnknown : e);
      return nullptr;
    }
    g_static_addr[device] = ptr;
  }
  return g_static_addr[device];
}
}  // namespace

extern "C" {

const char *h3b_last_error(void) { return g_error.c_str(); }

h3b_ctx *h3b_open(int device) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) {
    fail_cuda("cudaGetDeviceCount", e);
    return nullptr;
  }
  if (device < 0 || device >= count) {
    fail("device " + std::to_string(device) + " does not exist (" + std::to_string(count) + " CUDA devices)");
    return nullptr;
  }
  h3b_ctx *ctx = new h3b_ctx;
  ctx->device = device;
  auto bail = [&](const char *what, cudaError_t err) -> h3b_ctx * {
    fail_cuda(what, err);
    delete ctx;
    return nullptr;
  };
  if ((e = cudaSetDevice(device)) != cudaSuccess) return bail("cudaSetDevice", e);
  if ((e = cudaGetDeviceProperties(&ctx->prop, device)) != cudaSuccess) return bail("cudaGetDeviceProperties", e);
  if (ctx->prop.major != 10 || ctx->prop.minor != 0) {
    fail(std::string("device ") + ctx->prop.name + " is compute capability " + std::to_string(ctx->prop.major) + "." +
         std::to_string(ctx->prop.minor) + "; this library is built for 10.0 (sm_100a: tcgen05 kind::i8) only");
    delete ctx;
    return nullptr;
  }
  ctx->name = ctx->prop.name;
  if ((e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return bail("cudaStreamCreate", e);
  ctx->stream = ctx->own_stream;
  if ((e = cudaEventCreate(&ctx->ev_start)) != cudaSuccess) return bail("cudaEventCreate", e);
  if ((e = cudaEventCreate(&ctx->ev_end)) != cudaSuccess) return bail("cudaEventCreate", e);
  if ((e = cudaMalloc(&ctx->status_dev, sizeof(int))) != cudaSuccess) return bail("cudaMalloc", e);
  if ((e = cudaMemset(ctx->status_dev, 0, sizeof(int))) != cudaSuccess) return bail("cudaMemset", e);
  if ((e = cudaMallocHost(&ctx->status_host, sizeof(int))) != cudaSuccess) return bail("cudaMallocHost", e);
  *ctx->status_host = 0;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if ((e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q)) != cudaSuccess || !fn ||
      q != cudaDriverEntryPointSuccess) {
    if (e == cudaSuccess) e = cudaErrorUnknown;
    return bail("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", e);
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  if ((e = h3b::gemm_configure(device)) != cudaSuccess) return bail("cudaFuncSetAttribute(max dynamic shared memory)", e);
  if ((e = h3b::gemm_pair_configure()) != cudaSuccess) return bail("cudaFuncSetAttribute(max dynamic shared memory)", e);
  ctx->pair_stages = h3b::gemm_pair_pick_stages(ctx->prop.sharedMemPerBlockOptin, false);
  ctx->pair_stages_staged = h3b::gemm_pair_pick_stages(ctx->prop.sharedMemPerBlockOptin, true);
  ctx->pair_clusters = ctx->pair_stages >= 2 ? h3b::gemm_pair_max_clusters(ctx->pair_stages) : 0;
  cudaGetLastError();  // an occupancy query that failed must not poison the next launch check
  // the static scratch of h3b_gemm_w8a8_lora_noalloc is resolved (and thereby placed on this device) now, at set-up
  if (device < kMaxDevices && !static_scratch(device)) {
    delete ctx;
    return nullptr;
  }
  return ctx;
}

void h3b_close(h3b_ctx *ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
  if (ctx->ev_end) cudaEventDestroy(ctx->ev_end);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
}

const char *h3b_device_name(h3b_ctx *ctx) { return ctx ? ctx->name.c_str() : ""; }
uint64_t h3b_recommended_working_set(h3b_ctx *ctx) { return ctx ? ctx->prop.totalGlobalMem : 0; }
uint64_t h3b_max_buffer_length(h3b_ctx *ctx) { return ctx ? ctx->prop.totalGlobalMem : 0; }
int h3b_sm_count(h3b_ctx *ctx) { return ctx ? ctx->prop.multiProcessorCount : 0; }

int h3b_set_stream(h3b_ctx *ctx, void *cuda_stream) {
  if (!ctx) return fail("null context");
  ctx->stream = static_cast<cudaStream_t>(cuda_stream);
  return 0;
}

int h3b_use_own_stream(h3b_ctx *ctx) {
  if (!ctx) return fail("null context");
  ctx->stream = ctx->own_stream;
  return 0;
}

int h3b_set_launch_overlap(h3b_ctx *ctx, int on) {
  if (!ctx) return fail("null context");
  ctx->overlap = on != 0;
  return 0;
}

int h3b_rot_set_policy(h3b_ctx *ctx, int threads_target, int tma_stages, int chunk) {
  if (!ctx) return fail("null context");
  if (tma_stages < -1 || tma_stages > 4) return fail("rot policy: tma_stages must be -1 (off), 0 (automatic) or 1..4");
  if (chunk != 0 && chunk != 32 && chunk != 64) return fail("rot policy: chunk must be 0 (automatic), 32 or 64");
  ctx->rot_threads = threads_target;
  ctx->rot_stages = tma_stages;
  ctx->rot_chunk = chunk;
  return 0;
}

static int rot_enqueue(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out, float *sa, int M, int D,
                       int block, int mode, int out_hr, int scale_mode, const h3b::RotShardArgs *shard = nullptr) {
  if (!ctx) return fail("null context");
  if (shard && !(ctx->rot_stages >= 0 && h3b::rot_q8_tma_supported(x_dtype, D)))
    return fail("rot_q8: row maxima through peer memory need 16-bit inputs of at most 16384 channels");
  if (!x || (!out && scale_mode != 1) || (!out_hr && !sa)) return fail("rot_q8: null tensor argument");
  if (scale_mode < 0 || scale_mode > 2 || (scale_mode && out_hr)) return fail("rot_q8: bad scale mode");
  if (M <= 0 || D <= 0) return fail("rot_q8: M and D must be positive");
  if (block != 64 && block != 128 && block != 256) return fail("rot_q8: rotation block must be 64, 128 or 256");
  if (D % block) return fail("rot_q8: D " + std::to_string(D) + " is not a multiple of the rotation block " + std::to_string(block));
  if (mode != 0 && mode != 1) return fail("rot_q8: mode must be 0 or 1");
  const int esize = x_dtype == H3B_F32 ? 4 : (x_dtype == H3B_F16 || x_dtype == H3B_BF16) ? 2 : 0;
  if (!esize) return fail("rot_q8: input type must be bf16, f16 or f32");
  if (x_stride < (mode == 1 ? 2LL * D : D)) return fail("rot_q8: x_stride is smaller than the row");
  if (reinterpret_cast<uintptr_t>(x) % 16 || (x_stride * esize) % 16)
    return fail("rot_q8: input rows must be 16-byte aligned");
  if (out && reinterpret_cast<uintptr_t>(out) % 16) return fail("rot_q8: output must be 16-byte aligned");
  cudaEvent_t ps = nullptr;
  if (ctx->rot_stages >= 0 && h3b::rot_q8_tma_supported(x_dtype, D)) {
    // rows reach shared memory by TMA: the input seen as {64 channels, cols / 64 chunks, M rows}
    const uint64_t cols = mode == 1 ? 2ull * D : static_cast<uint64_t>(D);
    const CUtensorMap *map = ctx->tensor_map3(x, x_dtype, 64, cols / 64, M, 128, static_cast<uint64_t>(x_stride) * 2, 64,
                                              static_cast<uint32_t>(D / 64), 128);
    if (!map) return -1;
    if (ctx->before_launch(&ps)) return -1;
    const cudaError_t e = h3b::launch_rot_q8_tma(*map, x_dtype, out, sa, M, D, block, mode, out_hr, scale_mode, ctx->rot_stages,
                                                 ctx->rot_chunk, ctx->prop.multiProcessorCount, ctx->status_dev,
                                                 ctx->stream, ctx->overlap != 0 && !ctx->profile, shard);
    return ctx->after_launch("rot_q8 launch", e);
  }
  int target = ctx->rot_threads > 0 ? ctx->rot_threads : 256;
  if (target < 32) target = 32;
  if (target > 256) target = 256;
  int ch, threads;
  h3b::rot_q8_geometry(D, target, &ch, &threads);
  if (threads > 256) return fail("rot_q8: D " + std::to_string(D) + " exceeds the 32768 channels one CTA covers");
  if (ctx->before_launch(&ps)) return -1;
  const cudaError_t e = h3b::launch_rot_q8(x, x_dtype, x_stride, out, sa, M, D, block, mode, out_hr, scale_mode, target,
                                           ctx->prop.multiProcessorCount, ctx->stream);
  return ctx->after_launch("rot_q8 launch", e);
}

int h3b_rot_q8(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out, float *sa, int M, int D,
               int block, int mode, int out_hr) {
  return rot_enqueue(ctx, x, x_dtype, x_stride, out, sa, M, D, block, mode, out_hr, 0);
}

int h3b_rot_amax(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, float *amax, int M, int D, int block,
                 int mode) {
  return rot_enqueue(ctx, x, x_dtype, x_stride, nullptr, amax, M, D, block, mode, 0, 1);
}

int h3b_rot_q8_given_amax(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out, float *amax_to_scale,
                          int M, int D, int block, int mode) {
  return rot_enqueue(ctx, x, x_dtype, x_stride, out, amax_to_scale, M, D, block, mode, 0, 2);
}

int h3b_rot_amax_push(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, float *const *dst, int world, int M,
                      int D, int block, int mode) {
  if (!dst || world < 1 || world > h3b::kMaxPeers) return fail("rot_amax_push: 1 to 8 destinations");
  h3b::RotShardArgs sh = {};
  for (int i = 0; i < world; ++i) {
    if (!dst[i] || reinterpret_cast<uintptr_t>(dst[i]) % 4) return fail("rot_amax_push: null or misaligned destination");
    sh.amax_dst[i] = dst[i];
  }
  sh.n_dst = world; sh.amax_slots = 1; sh.scale_out = dst[0];
  return rot_enqueue(ctx, x, x_dtype, x_stride, nullptr, dst[0], M, D, block, mode, 0, 1, &sh);
}

int h3b_rot_q8_given_amax_slots(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out, const float *slots,
                                int64_t slot_stride, int world, float *scale, int M, int D, int block, int mode) {
  if (!slots || !scale || world < 1 || world > h3b::kMaxPeers || slot_stride < M)
    return fail("rot_q8_given_amax_slots: need 1 to 8 slots of at least M maxima and a scale buffer");
  h3b::RotShardArgs sh = {};
  sh.n_dst = 0; sh.amax_slots = world; sh.amax_slot_stride = slot_stride; sh.scale_out = scale;
  return rot_enqueue(ctx, x, x_dtype, x_stride, out, const_cast<float *>(slots), M, D, block, mode, 0, 2, &sh);
}

int h3b_norm_mod_q8(h3b_ctx *ctx, float *x, int64_t x_stride, const float *mod, int64_t mod_stride,
                    const uint8_t *rtype, void *out, float *sa, int M, int D, int block, float eps, int ln, int out_kind,
                    const float *y, const float *post) {
  if (!ctx) return fail("null context");
  if (!x || !mod || !rtype || !out) return fail("norm_mod_q8: null tensor argument");
  if (out_kind < 0 || out_kind > 3) return fail("norm_mod_q8: out_kind must be 0 (int8), 1 (fp32), 2 (fp16) or 3 (rotated fp16)");
  if (out_kind == 0 && !sa) return fail("norm_mod_q8: int8 output needs the row-scale buffer");
  if (M <= 0 || D <= 0) return fail("norm_mod_q8: M and D must be positive");
  if (block != 64 && block != 128 && block != 256) return fail("norm_mod_q8: rotation block must be 64, 128 or 256");
  if (D % block) return fail("norm_mod_q8: D " + std::to_string(D) + " is not a multiple of the rotation block " + std::to_string(block));
  if ((post != nullptr) != (y != nullptr)) return fail("norm_mod_q8: y and post go together");
  if (ln && post) return fail("norm_mod_q8: LayerNorm excludes the fused residual update");
  if (x_stride < D || mod_stride < 2LL * D) return fail("norm_mod_q8: x_stride / mod_stride smaller than the row");
  if (D > (post ? 16384 : 32768)) return fail("norm_mod_q8: D exceeds what one CTA covers (32768; 16384 with the residual update)");
  if (reinterpret_cast<uintptr_t>(x) % 16 || (x_stride * 4) % 16 || reinterpret_cast<uintptr_t>(mod) % 16 ||
      (mod_stride * 4) % 16 || reinterpret_cast<uintptr_t>(out) % 16 ||
      (y && reinterpret_cast<uintptr_t>(y) % 16) || (post && reinterpret_cast<uintptr_t>(post) % 16))
    return fail("norm_mod_q8: tensors must be 16-byte aligned with row strides that are multiples of 16 bytes");
  cudaEvent_t ps = nullptr;
  if (!post && ctx->rot_stages >= 0 && h3b::norm_mod_q8_tma_supported(D) && mod_stride % 32 == 0) {
    // rows reach shared memory by TMA: x seen as {32 floats, x_stride / 32 lines, M rows}
    const CUtensorMap *map = ctx->tensor_map3(x, h3b::kDtypeF32, 32, static_cast<uint64_t>(D) / 32, M, 128,
                                              static_cast<uint64_t>(x_stride) * 4, 32, static_cast<uint32_t>(D / 32), 128);
    if (!map) return -1;
    const CUtensorMap map_x = *map;  // the cache may move when the second descriptor is inserted
    // the modulation table seen the same way: {32 floats, mod_stride / 32 lines, up to 256 row types}
    const CUtensorMap *mmap = ctx->tensor_map3(mod, h3b::kDtypeF32, 32, static_cast<uint64_t>(mod_stride) / 32, 256, 128,
                                               static_cast<uint64_t>(mod_stride) * 4, 32, static_cast<uint32_t>(D / 32), 128);
    if (!mmap) return -1;
    if (ctx->before_launch(&ps)) return -1;
    const cudaError_t e = h3b::launch_norm_mod_q8_tma(map_x, *mmap, mod, mod_stride, rtype, out, sa, M, D, block, eps, ln, out_kind,
                                                      ctx->rot_stages, ctx->rot_chunk, ctx->prop.multiProcessorCount,
                                                      ctx->status_dev, ctx->stream);
    return ctx->after_launch("norm_mod_q8 launch", e);
  }
  if (ctx->before_launch(&ps)) return -1;
  const cudaError_t e = h3b::launch_norm_mod_q8(x, x_stride, mod, mod_stride, rtype, out, sa, M, D, block, eps, ln, out_kind,
                                                y, post, ctx->stream);
  return ctx->after_launch("norm_mod_q8 launch", e);
}

int h3b_dequant_i32(h3b_ctx *ctx, const int32_t *acc, int64_t acc_stride, const float *sa, const float *sw,
                    const float *bias, void *C, int c_dtype, int64_t c_stride, int M, int N) {
  if (!ctx) return fail("null context");
  if (!acc || !sa || !sw || !C) return fail("dequant: null tensor argument");
  if (M <= 0 || N <= 0 || acc_stride < N || c_stride < N) return fail("dequant: bad sizes");
  if (c_dtype != H3B_BF16 && c_dtype != H3B_F16 && c_dtype != H3B_F32) return fail("dequant: output type must be bf16, f16 or f32");
  cudaEvent_t ps = nullptr;
  if (ctx->before_launch(&ps)) return -1;
  const cudaError_t e = h3b::launch_dequant_i32(acc, acc_stride, sa, sw, bias, C, c_dtype, c_stride, M, N,
                                                ctx->prop.multiProcessorCount, ctx->stream);
  return ctx->after_launch("dequant launch", e);
}

int h3b_gemm_set_policy(h3b_ctx *ctx, int tile_n, int band, int pair) {
  if (!ctx) return fail("null context");
  if (pair < -1 || pair > 1) return fail("gemm policy: pair must be -1 (never), 0 (automatic) or 1 (whenever possible)");
  ctx->pair_mode = pair;
  if (tile_n != 0 && tile_n != 32 && tile_n != 64 && tile_n != 128 && tile_n != 256)
    return fail("gemm policy: tile_n must be 0, 32, 64, 128 or 256");
  if (band < 0) return fail("gemm policy: band must be >= 0");
  ctx->tile_n_override = tile_n;
  ctx->band_override = band;
  return 0;
}

int h3b_gemm_set_store_mode(h3b_ctx *ctx, int mode) {
  if (!ctx) return fail("null context");
  if (mode < -1 || mode > 1) return fail("gemm store mode: -1 (direct stores), 0 (automatic) or 1 (staged whenever possible)");
  ctx->store_mode = mode;
  return 0;
}

int h3b_gemm_tile_n(h3b_ctx *ctx, int N, int /*lora*/) {
  if (ctx && ctx->tile_n_override) return ctx->tile_n_override;
  if (N <= 32) return 32;
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  if (N % 256 == 0 || N >= 2048) return 256;
  return 128;
}

// Checks the arguments of one product and enqueues it. cached_maps: TMA descriptors come from (and go into) the
// context's cache; false builds them on the stack: no device allocation, and no host allocation either outside
// profile mode (which records a time per launch) and error messages. check_only: every check, no launch.
static int gemm_enqueue(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                        const float *sw, const float *sa, const float *bias, void *C, int c_dtype, int64_t c_stride,
                        int M, int N, int K, const void *lora_T, int64_t t_stride, const void *lora_B,
                        int64_t b_stride, int R, const int32_t *lora_ranges, bool cached_maps,
                        const uint8_t *rtype = nullptr, const float *gate = nullptr, int64_t g_stride = 0,
                        void *const *push_slots = nullptr, int push_world = 0, int push_rows = 0,
                        bool check_only = false) {
  if (!ctx) return fail("null context");
  const bool push = push_slots != nullptr;
  if (push) {
    if (push_world < 1 || push_world > h3b::kMaxPeers) return fail("gemm (push): 1 to 8 GPUs");
    if (push_rows <= 0 || push_rows % 128) return fail("gemm (push): every GPU owns a multiple of 128 rows");
    if (static_cast<long long>(push_rows) * push_world != M) return fail("gemm (push): M must equal rows_per_gpu x world");
    if (c_dtype != H3B_I32 && c_dtype != H3B_BF16) return fail("gemm (push): staging holds int32 accumulators or bf16 partials");
    if (N % 32) return fail("gemm (push): N must be a multiple of 32");
    if ((c_stride * (c_dtype == H3B_I32 ? 4 : 2)) % 16) return fail("gemm (push): staging rows must be multiples of 16 bytes");
    for (int i = 0; i < push_world; ++i)
      if (!push_slots[i] || reinterpret_cast<uintptr_t>(push_slots[i]) % 16) return fail("gemm (push): null or misaligned slot");
    if (lora_T || gate) return fail("gemm (push): no low-rank term and no gated epilogue on a row-parallel layer");
    C = push_slots[0];
  }
  if (!A || !W || !C) return fail("gemm: null tensor argument");
  if (M <= 0 || N <= 0 || K <= 0) return fail("gemm: M, N and K must be positive");
  const bool raw = c_dtype == H3B_I32;
  if (!raw && c_dtype != H3B_BF16 && c_dtype != H3B_F16 && c_dtype != H3B_F32)
    return fail("gemm: output type must be bf16, f16, f32 or i32");
  if (!raw && (!sw || !sa)) return fail("gemm: int8 products need row scales (sa) and column scales (sw)");
  if (a_stride < K || w_stride < K) return fail("gemm: a_stride / w_stride smaller than K");
  if (c_stride < N) return fail("gemm: c_stride smaller than N");
  if (reinterpret_cast<uintptr_t>(A) % 16 || reinterpret_cast<uintptr_t>(W) % 16 || a_stride % 16 || w_stride % 16)
    return fail("gemm: A and W must be 16-byte aligned with row strides that are multiples of 16 bytes");
  const bool lora = !raw && lora_T != nullptr;
  if (lora) {
    if (!lora_B) return fail("gemm: low-rank term needs both T and B");
    if (R <= 0 || R % 32 || R > 128) return fail("gemm: low-rank R must be a multiple of 32, at most 128");
    if (t_stride < R || b_stride < R) return fail("gemm: t_stride / b_stride smaller than R");
    if (reinterpret_cast<uintptr_t>(lora_T) % 16 || reinterpret_cast<uintptr_t>(lora_B) % 16 || (t_stride * 2) % 16 ||
        (b_stride * 2) % 16)
      return fail("gemm: T and B must be 16-byte aligned with row strides that are multiples of 16 bytes");
  }
  // CTA pairs (256 x 256 tiles, the W tile shared across the pair: a third less traffic from L2 and through shared
  // memory per multiply) wherever a product has at least one whole pair tile and neither a low-rank term nor the
  // row-parallel push, which only the single-CTA kernel (128 x tile_n tiles) implements. Under the board's power cap
  // the saved data movement is what counts: measured on the 33B-class shapes 2.67-2.83 POPS against 2.54-2.61.
  const bool pair_fits = M >= 256 && N >= 256;
  // a low-rank term's rank ranges come per column tile: pairs need the table of 256-column tiles
  const bool pair = !push && ctx->pair_clusters > 0 && !ctx->tile_n_override &&
                    (!lora || h3b_gemm_tile_n(ctx, N, 1) == 256) &&
                    (ctx->pair_mode == 1 || (ctx->pair_mode == 0 && pair_fits));
  // Staged stores (the epilogue writes 16-bit outputs to shared memory and TMA stores them) cost two of the six ring
  // stages, about 1.5 k cycles of operand waits per tile, and shorten the epilogue by about 5 k cycles. The epilogue is
  // hidden behind the next tile either way (with a low-rank term too: its int32 accumulator is handed back before any
  // arithmetic), so they pay where only the last, exposed epilogue counts - launches of at most three tiles per pair
  // with a short K (+3.5 % at 4096 x 3072 x 3072; -2.5 % on the 33B-class and Z-Image blocks) - and for very tall
  // products, whose output no longer fits L2 (M = 66560: +1 %).
  const bool can_stage = pair && (c_dtype == H3B_BF16 || c_dtype == H3B_F16) && gate == nullptr && ctx->pair_stages_staged >= 2 &&
                         reinterpret_cast<uintptr_t>(C) % 16 == 0 && (c_stride * 2) % 16 == 0;
  const long long pair_tiles = ((M + 255LL) / 256) * ((N + 255LL) / 256);
  const bool few_tiles = pair && pair_tiles <= 3LL * ctx->pair_clusters && K <= 4096;
  const bool staged = can_stage && (ctx->store_mode == 1 || (ctx->store_mode == 0 && (few_tiles || M >= 49152)));
  const int bn = pair ? 128 : h3b_gemm_tile_n(ctx, N, lora);  // rows of W one CTA stages per K block
  const int stages = pair ? (staged ? ctx->pair_stages_staged : ctx->pair_stages)
                          : h3b::gemm_pick_stages(bn, lora ? R : 0, ctx->prop.sharedMemPerBlockOptin, push);
  if (stages < 2) return fail("gemm: tile does not fit the device's shared memory");

  h3b::GemmLaunch g;
  memset(&g, 0, sizeof g);
  const CUtensorMap *m;
  CUtensorMap local;
  if (!(m = ctx->map2(cached_maps, &local, A, h3b::kDtypeI8, K, M, a_stride, 128, 128, 128))) return -1;
  g.map_a = *m;
  if (!(m = ctx->map2(cached_maps, &local, W, h3b::kDtypeI8, K, N, w_stride, 128, bn, 128))) return -1;
  g.map_w = *m;
  if (lora) {
    if (!(m = ctx->map2(cached_maps, &local, lora_T, h3b::kDtypeF16, R, M, t_stride * 2, 32, 128, 64))) return -1;
    g.map_t = *m;
    if (!(m = ctx->map2(cached_maps, &local, lora_B, h3b::kDtypeF16, R, N, b_stride * 2, 32, bn, 64))) return -1;
    g.map_b = *m;
  }
  // One accumulator pair leaves a low-rank product's epilogue exposed: sixteen warps (four per TMEM lane quarter, 64
  // columns each) read the accumulators out in a quarter of the time four would take. Measured on M = 66560,
  // 6144 -> 18432, rank 64, single launches: 6.11 / 5.95 / 5.25 ms with 4 / 8 / 16 warps against 4.7 ms without a term.
  if (staged) {
    if (!(m = ctx->map2(cached_maps, &local, C, c_dtype, N, M, c_stride * 2, 64, 32, 128))) return -1;
    g.map_c = *m;
    g.tma_store = 1;
  }
  if (gate != nullptr) {
    if (!rtype) return fail("gemm: the gated-residual epilogue needs the row types");
    if (c_dtype != H3B_F32) return fail("gemm: the gated-residual epilogue accumulates into an fp32 residual stream");
    if (g_stride < N) return fail("gemm: g_stride smaller than N");
  }
  g.rtype = rtype; g.gate = gate; g.g_stride = g_stride;
  if (push) {
    for (int i = 0; i < push_world; ++i) g.peer_c[i] = push_slots[i];
    g.peer_rows = push_rows;
  }
  g.sw = sw; g.sa = sa; g.bias = raw ? nullptr : bias; g.c = C; g.ranges = lora ? lora_ranges : nullptr;
  g.c_stride = c_stride; g.c_dtype = c_dtype; g.M = M; g.N = N; g.K = K; g.R = lora ? R : 0; g.bn = bn;
  g.acc_stages = (lora && (bn == 256 || pair)) ? 1 : 2;
  const int tile_m = pair ? 256 : 128, tile_n = pair ? 256 : bn;
  const int m_tiles = (M + tile_m - 1) / tile_m, n_tiles = (N + tile_n - 1) / tile_n;
  int band = ctx->band_override;
  if (band <= 0) {
    // keep the A band (band x tile_m rows x K bytes) inside L2 while W streams through once per band; measured on
    // M = 17408: the product is fastest with 27-36 MB bands and loses 6-15 % from 53 MB on
    const long long budget = 32LL << 20;
    band = static_cast<int>(budget / (static_cast<long long>(tile_m) * K));
    if (band < (pair ? 2 : 4)) band = pair ? 2 : 4;
  }
  // push: the tiles in flight at any moment should span every owner's rows, so that no GPU's incoming links
  // become the bottleneck while others idle: one band over all rows (A's K shard is small enough for L2)
  if (push && static_cast<long long>(M) * K <= (64LL << 20)) band = m_tiles;
  if (band > m_tiles) band = m_tiles;
  g.band = band;
  const long long tiles = static_cast<long long>(m_tiles) * n_tiles;
  g.status = ctx->status_dev;
  g.overlap = (ctx->overlap != 0 && !ctx->profile) ? 1 : 0;
  if (check_only) return 0;

  cudaEvent_t ps = nullptr;
  if (ctx->before_launch(&ps)) return -1;
  if (pair) {
    const int clusters = static_cast<int>(tiles < ctx->pair_clusters ? tiles : ctx->pair_clusters);
    g.grid = 2 * clusters;
    return ctx->after_launch("gemm launch", h3b::launch_gemm_w8a8_pair(g, stages, clusters, ctx->stream));
  }
  g.grid = static_cast<int>(tiles < ctx->prop.multiProcessorCount ? tiles : ctx->prop.multiProcessorCount);
  const cudaError_t e = h3b::launch_gemm_w8a8(g, stages, ctx->stream);
  return ctx->after_launch("gemm launch", e);
}

int h3b_gemm_w8a8(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                  const float *sw, const float *sa, const float *bias, void *C, int c_dtype, int64_t c_stride,
                  int M, int N, int K, const void *lora_T, int64_t t_stride, const void *lora_B, int64_t b_stride,
                  int R, const int32_t *lora_ranges) {
  return gemm_enqueue(ctx, A, a_stride, W, w_stride, sw, sa, bias, C, c_dtype, c_stride, M, N, K, lora_T, t_stride,
                      lora_B, b_stride, R, lora_ranges, true);
}

int h3b_gemm_w8a8_gated(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                        const float *sw, const float *sa, const float *bias, float *X, int64_t c_stride, int M, int N,
                        int K, const uint8_t *rtype, const float *gate, int64_t g_stride, const void *lora_T,
                        int64_t t_stride, const void *lora_B, int64_t b_stride, int R, const int32_t *lora_ranges) {
  if (!gate) return fail("gemm (gated): null gate table");
  return gemm_enqueue(ctx, A, a_stride, W, w_stride, sw, sa, bias, X, H3B_F32, c_stride, M, N, K, lora_T, t_stride, lora_B,
                      b_stride, R, lora_ranges, true, rtype, gate, g_stride);
}

// ---- row-parallel layers over the GPUs of one node -----------------------------------------------------------------
void *h3b_peer_alloc(h3b_ctx *ctx, uint64_t bytes) {
  if (!ctx || bytes == 0) {
    fail("peer_alloc: null context or zero size");
    return nullptr;
  }
  if (ctx->make_current()) return nullptr;
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the zeros are in place before the address leaves this call
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    fail_cuda("peer_alloc", e);
    return nullptr;
  }
  return p;
}

int h3b_peer_free(h3b_ctx *ctx, void *ptr) {
  if (!ctx) return fail("null context");
  if (ctx->make_current()) return -1;
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : fail_cuda("peer_free", e);
}

int h3b_peer_export(h3b_ctx *ctx, void *ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");
  if (!ctx || !ptr || !handle) return fail("peer_export: null argument");
  if (ctx->make_current()) return -1;
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return fail_cuda("cudaIpcGetMemHandle", e);
  memcpy(handle, &h, 64);
  return 0;
}

void *h3b_peer_import(h3b_ctx *ctx, const unsigned char handle[64]) {
  if (!ctx || !handle) {
    fail("peer_import: null argument");
    return nullptr;
  }
  if (ctx->make_current()) return nullptr;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void *p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fail_cuda("cudaIpcOpenMemHandle", e);
    return nullptr;
  }
  return p;
}

int h3b_peer_unmap(h3b_ctx *ctx, void *ptr) {
  if (!ctx) return fail("null context");
  if (ctx->make_current()) return -1;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : fail_cuda("cudaIpcCloseMemHandle", e);
}

int h3b_peer_sync(h3b_ctx *ctx, void *const *flags, int rank, int world, uint32_t epoch, int mode) {
  if (!ctx || !flags) return fail("peer_sync: null argument");
  if (world < 1 || world > h3b::kMaxPeers || rank < 0 || rank >= world) return fail("peer_sync: bad rank / world");
  if (mode < 0 || mode > 2) return fail("peer_sync: mode must be 0 (signal and wait), 1 (signal) or 2 (wait)");
  h3b::PeerSync p = {};
  for (int i = 0; i < world; ++i) {
    if (!flags[i] || reinterpret_cast<uintptr_t>(flags[i]) % 4) return fail("peer_sync: null or misaligned flag array");
    p.flags[i] = static_cast<unsigned int *>(flags[i]);
  }
  p.rank = rank; p.world = world; p.mode = mode; p.epoch = epoch; p.status = ctx->status_dev;
  p.limit_cycles = 2000000000LL;  // about a second at the part's clocks
  cudaEvent_t ps = nullptr;
  if (ctx->before_launch(&ps)) return -1;
  return ctx->after_launch("peer_sync launch", h3b::launch_peer_sync(p, ctx->stream));
}

int h3b_gemm_w8a8_push(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                       const float *sw, const float *sa, void *const *slots, int world, int rows_per_gpu,
                       int stage_dtype, int64_t stage_stride, int M, int N, int K) {
  if (!slots) return fail("gemm (push): null slot table");
  return gemm_enqueue(ctx, A, a_stride, W, w_stride, sw, sa, nullptr, nullptr, stage_dtype, stage_stride, M, N, K, nullptr, 0,
                      nullptr, 0, 0, nullptr, true, nullptr, nullptr, 0, slots, world, rows_per_gpu);
}

static int reduce_enqueue(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride, int stage_dtype,
                          int world, const float *sa, const float *sw, const float *bias, void *const *outs, int n_out,
                          int c_dtype, int64_t c_stride, int rows, int N, int row0, const uint8_t *rtype,
                          const float *gate, int64_t g_stride, const float *low = nullptr, int64_t low_stride = 0) {
  if (!ctx) return fail("null context");
  if (!stage || !outs) return fail("reduce_dequant: null tensor argument");
  if (world < 1 || world > h3b::kMaxPeers || n_out < 1 || n_out > h3b::kMaxPeers) return fail("reduce_dequant: 1 to 8 slots and outputs");
  if (stage_dtype != H3B_I32 && stage_dtype != H3B_BF16) return fail("reduce_dequant: staging holds int32 or bf16");
  if (stage_dtype == H3B_I32 && (!sa || !sw)) return fail("reduce_dequant: int32 partials need the row and column scales");
  if (c_dtype != H3B_BF16 && c_dtype != H3B_F16 && c_dtype != H3B_F32) return fail("reduce_dequant: output type must be bf16, f16 or f32");
  if (rows <= 0 || N <= 0 || N % 8 || stage_stride < N || c_stride < N || row0 < 0) return fail("reduce_dequant: bad sizes (N must be a multiple of 8)");
  const int ss = stage_dtype == H3B_I32 ? 4 : 2, cs = c_dtype == H3B_F32 ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(stage) % 16 || (stage_stride * ss) % 16 || (slot_stride * ss) % 16 || (c_stride * cs) % 16 ||
      (sw && reinterpret_cast<uintptr_t>(sw) % 16) || (bias && reinterpret_cast<uintptr_t>(bias) % 16))
    return fail("reduce_dequant: tensors must be 16-byte aligned with strides that are multiples of 16 bytes");
  h3b::ReduceLaunch r = {};
  r.stage = stage; r.slot_stride = slot_stride; r.stage_stride = stage_stride; r.stage_dtype = stage_dtype; r.world = world;
  r.sa = sa; r.sw = sw; r.bias = bias; r.n_out = n_out; r.c_stride = c_stride; r.c_dtype = c_dtype; r.rows = rows; r.N = N;
  r.row0 = row0;
  if (low) {
    if (low_stride < N || (low_stride * 4) % 16 || reinterpret_cast<uintptr_t>(low) % 16)
      return fail("reduce_dequant: the low-rank term's rows must be 16-byte aligned and at least N long");
    r.low = low; r.low_stride = low_stride;
  }
  r.status = ctx->status_dev;
  if (gate) {
    if (!rtype) return fail("reduce_dequant (gated): null row types");
    if (g_stride < N || (g_stride * 4) % 16 || reinterpret_cast<uintptr_t>(gate) % 16) return fail("reduce_dequant (gated): gate rows must be 16-byte aligned and at least N long");
    r.rtype = rtype; r.gate = gate; r.g_stride = g_stride;
  }
  for (int i = 0; i < n_out; ++i) {
    if (!outs[i] || reinterpret_cast<uintptr_t>(outs[i]) % 16) return fail("reduce_dequant: null or misaligned output");
    r.out[i] = outs[i];
  }
  cudaEvent_t ps = nullptr;
  if (ctx->before_launch(&ps)) return -1;
  return ctx->after_launch("reduce_dequant launch", h3b::launch_reduce_dequant(r, ctx->prop.multiProcessorCount, ctx->stream));
}

int h3b_reduce_dequant(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride, int stage_dtype,
                       int world, const float *sa, const float *sw, const float *bias, void *const *outs, int n_out,
                       int c_dtype, int64_t c_stride, int rows, int N, int row0) {
  return reduce_enqueue(ctx, stage, slot_stride, stage_stride, stage_dtype, world, sa, sw, bias, outs, n_out, c_dtype,
                        c_stride, rows, N, row0, nullptr, nullptr, 0);
}

int h3b_reduce_dequant_low(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride, int stage_dtype,
                           int world, const float *sa, const float *sw, const float *bias, const float *low,
                           int64_t low_stride, void *const *outs, int n_out, int c_dtype, int64_t c_stride, int rows, int N,
                           int row0, const uint8_t *rtype, const float *gate, int64_t g_stride) {
  if (!low) return fail("reduce_dequant_low: null low-rank term");
  return reduce_enqueue(ctx, stage, slot_stride, stage_stride, stage_dtype, world, sa, sw, bias, outs, n_out,
                        gate ? H3B_F32 : c_dtype, c_stride, rows, N, row0, rtype, gate, g_stride, low, low_stride);
}

int h3b_reduce_dequant_gated(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride, int stage_dtype,
                             int world, const float *sa, const float *sw, const float *bias, float *X, int64_t c_stride,
                             int rows, int N, int row0, const uint8_t *rtype, const float *gate, int64_t g_stride) {
  if (!gate) return fail("reduce_dequant (gated): null gate table");
  void *outs[1] = {X};
  return reduce_enqueue(ctx, stage, slot_stride, stage_stride, stage_dtype, world, sa, sw, bias, outs, 1, H3B_F32, c_stride,
                        rows, N, row0, rtype, gate, g_stride);
}

int h3b_gemm_w8a8_lora_noalloc(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                               const float *sw, const float *sa, const float *bias, void *C, int c_dtype,
                               int64_t c_stride, int M, int N, int K, const int8_t *lora_A, int64_t la_stride,
                               const float *lora_sw, const void *lora_B, int64_t b_stride, int R,
                               const int32_t *lora_ranges) {
  if (!ctx) return fail("null context");
  if (!lora_A || !lora_sw || !lora_B) return fail("no-alloc product: the low-rank term needs A codes, A scales and B");
  if (c_dtype == H3B_I32) return fail("no-alloc product: raw accumulators carry no low-rank term; use h3b_gemm_w8a8");
  if (M <= 0 || R <= 0 || R % 32 || R > 128) return fail("no-alloc product: R must be a multiple of 32, at most 128");
  const unsigned long long need = static_cast<unsigned long long>(M) * static_cast<unsigned long long>(R);
  if (need > H3B_NOALLOC_MAX_T_VALUES)
    return fail("no-alloc product: M x R = " + std::to_string(need) + " fp16 values exceed the library's static scratch of " +
                std::to_string(static_cast<unsigned long long>(H3B_NOALLOC_MAX_T_VALUES)) +
                " (8 MiB); split the rows or use h3b_gemm_w8a8 with your own T buffer");
  if (ctx->make_current()) return -1;
  void *T = static_scratch(ctx->device);
  if (!T) return -1;
  // both products' arguments are checked before the first launch: a refused call leaves the shared array untouched
  if (gemm_enqueue(ctx, A, a_stride, lora_A, la_stride, lora_sw, sa, nullptr, T, H3B_F16, R, M, R, K, nullptr, 0, nullptr,
                   0, 0, nullptr, false, nullptr, nullptr, 0, nullptr, 0, 0, true) ||
      gemm_enqueue(ctx, A, a_stride, W, w_stride, sw, sa, bias, C, c_dtype, c_stride, M, N, K, T, R, lora_B, b_stride, R,
                   lora_ranges, false, nullptr, nullptr, 0, nullptr, 0, 0, true))
    return -1;
  // T[m][j] = fp16(acc * sa[m] * lora_sw[j]) for every one of the M rows and R columns: the whole region the main
  // product reads is overwritten, so nothing of an earlier call survives into this one and nothing needs clearing.
  if (gemm_enqueue(ctx, A, a_stride, lora_A, la_stride, lora_sw, sa, nullptr, T, H3B_F16, R, M, R, K, nullptr, 0, nullptr,
                   0, 0, nullptr, false))
    return -1;
  return gemm_enqueue(ctx, A, a_stride, W, w_stride, sw, sa, bias, C, c_dtype, c_stride, M, N, K, T, R, lora_B, b_stride,
                      R, lora_ranges, false);
}

int h3b_selftest_expire_wait(h3b_ctx *ctx) {
  if (!ctx) return fail("null context");
  cudaEvent_t ps = nullptr;
  if (ctx->before_launch(&ps)) return -1;
  // about a millisecond at the part's clocks: long enough to be a real wait, short enough for a test
  return ctx->after_launch("self-test launch", h3b::launch_expire_wait(ctx->status_dev, 2000000LL, ctx->stream));
}

int h3b_mma_rate_probe(h3b_ctx *ctx, int pair, int iters, double out[5]) {
  if (!ctx || !out) return fail("mma_rate_probe: null argument");
  if (iters < 1 || iters > 4000000) return fail("mma_rate_probe: iters must be in [1, 4000000]");
  if (ctx->make_current()) return -1;
  int ctas = ctx->prop.multiProcessorCount;
  unsigned long long *cycles = nullptr;
  cudaError_t e = cudaMalloc(&cycles, sizeof(unsigned long long) * ctas);
  if (e != cudaSuccess) return fail_cuda("mma_rate_probe: cudaMalloc", e);
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  std::vector<unsigned long long> host(ctas, 0ull);
  float ms = 0;
  int rc = 0;
  if ((e = cudaEventCreate(&t0)) != cudaSuccess || (e = cudaEventCreate(&t1)) != cudaSuccess ||
      (e = cudaMemsetAsync(cycles, 0, sizeof(unsigned long long) * ctas, ctx->stream)) != cudaSuccess ||
      (e = cudaEventRecord(t0, ctx->stream)) != cudaSuccess ||
      (e = h3b::launch_mma_probe(pair != 0, iters, &ctas, ctx->status_dev, cycles, ctx->stream)) != cudaSuccess ||
      (e = cudaEventRecord(t1, ctx->stream)) != cudaSuccess || (e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess ||
      (e = cudaEventElapsedTime(&ms, t0, t1)) != cudaSuccess ||
      (e = cudaMemcpy(host.data(), cycles, sizeof(unsigned long long) * ctas, cudaMemcpyDeviceToHost)) != cudaSuccess)
    rc = fail_cuda("mma_rate_probe", e);
  if (t0) cudaEventDestroy(t0);
  if (t1) cudaEventDestroy(t1);
  cudaFree(cycles);
  if (rc) return rc;
  ++ctx->launches;
  unsigned long long worst = 0;
  for (int i = 0; i < ctas; ++i) {
    if (host[i] == 0) return fail("mma_rate_probe: a CTA's wait for its last instruction ran out");
    if (host[i] > worst) worst = host[i];
  }
  const double ops_per_cta = 2.0 * 128 * 256 * 32 * 4.0 * iters;  // each SM multiplies 128 x 256 x 32 per instruction
  out[0] = ms * 1e-3;
  out[1] = static_cast<double>(worst);
  out[2] = ops_per_cta / static_cast<double>(worst);
  out[3] = ops_per_cta * ctas / (ms * 1e-3) / 1e12;
  out[4] = ctas;
  return 0;
}

void h3b_commit(h3b_ctx *) {}

double h3b_wait(h3b_ctx *ctx) {
  if (!ctx) {
    fail("null context");
    return -1.0;
  }
  if (ctx->make_current()) return -1.0;
  cudaError_t e;
  double seconds = 0.0;
  if ((e = cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream)) != cudaSuccess) {
    fail_cuda("status read", e);
    return -1.0;
  }
  if (ctx->timing_open) {
    if ((e = cudaEventRecord(ctx->ev_end, ctx->stream)) != cudaSuccess) {
      fail_cuda("cudaEventRecord", e);
      return -1.0;
    }
  }
  if ((e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess) {
    ctx->timing_open = false;
    fail_cuda("GPU work failed", e);
    return -1.0;
  }
  if (ctx->timing_open) {
    float ms = 0;
    if (cudaEventElapsedTime(&ms, ctx->ev_start, ctx->ev_end) == cudaSuccess) seconds = ms * 1e-3;
    ctx->timing_open = false;
  }
  if (*ctx->status_host != 0) {
    const int code = *ctx->status_host;
    *ctx->status_host = 0;
    cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    fail(std::string("GPU kernel gave up: ") + status_text(code));
    return -1.0;
  }
  return seconds;
}

void h3b_set_profile(h3b_ctx *ctx, int on) {
  if (!ctx) return;
  h3b_wait(ctx);
  ctx->profile = on != 0;
  ctx->prof.clear();
}

int h3b_profile_take(h3b_ctx *ctx, double *seconds, int max) {
  if (!ctx || !seconds || max <= 0) return 0;
  const int n = static_cast<int>(ctx->prof.size()) < max ? static_cast<int>(ctx->prof.size()) : max;
  for (int i = 0; i < n; ++i) seconds[i] = ctx->prof[i];
  ctx->prof.erase(ctx->prof.begin(), ctx->prof.begin() + n);
  return n;
}

uint64_t h3b_launch_count(h3b_ctx *ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
