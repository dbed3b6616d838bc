// Shared helpers of the sm_100a kernels: error reporting through return codes and a
// per-library message, element types, conversions, warp and block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define TS_EXPORT extern "C" __attribute__((visibility("default")))

// element type codes shared with the Python bindings
enum TsDtype : int { TS_F32 = 0, TS_BF16 = 1 };

static thread_local char ts_error_message[512] = "";

static inline int ts_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(ts_error_message, sizeof(ts_error_message), fmt, ap);
  va_end(ap);
  return 1;
}

#define TS_REQUIRE(cond, ...) \
  do {                        \
    if (!(cond)) return ts_fail(__VA_ARGS__); \
  } while (0)

#define TS_CHECK_LAUNCH(name)                                                   \
  do {                                                                          \
    cudaError_t e_ = cudaGetLastError();                                        \
    if (e_ != cudaSuccess) return ts_fail("%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

#ifdef TS_TIMELINE
// A build for looking at how the kernels of a step overlap: thread 0 of every block records the
// GPU's global timer when the block starts (tag 0), when its wait for the predecessor returns
// (tag 1) and wherever a kernel calls timeline_mark itself.  ts_timeline_read copies the records
// out.  Product builds compile none of it.
struct TimelineRecord {
  unsigned long long ns;
  int sm, tag, grid_x, grid_y, grid_z, block_x, block_y, block_z, threads, pad;
};
constexpr unsigned TIMELINE_CAPACITY = 1u << 17;
static __device__ TimelineRecord g_timeline[TIMELINE_CAPACITY];
static __device__ unsigned g_timeline_count;
// a mark of the calling thread, whichever it is, with a value of its own (a loop count, say)
__device__ __forceinline__ void timeline_mark_thread(int tag, int value) {
  unsigned long long ns;
  unsigned sm;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  const unsigned i = atomicAdd(&g_timeline_count, 1u);
  if (i < TIMELINE_CAPACITY)
    g_timeline[i] = TimelineRecord{ns, (int)sm, tag, (int)gridDim.x, (int)gridDim.y, (int)gridDim.z,
                                   (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z,
                                   (int)(blockDim.x * blockDim.y * blockDim.z), value};
}
__device__ __forceinline__ void timeline_mark(int tag) {
  if (threadIdx.x | threadIdx.y | threadIdx.z) return;
  unsigned long long ns;
  unsigned sm;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  const unsigned i = atomicAdd(&g_timeline_count, 1u);
  if (i < TIMELINE_CAPACITY)
    g_timeline[i] = TimelineRecord{ns, (int)sm, tag, (int)gridDim.x, (int)gridDim.y, (int)gridDim.z,
                                   (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z,
                                   (int)(blockDim.x * blockDim.y * blockDim.z), 0};
}
#define TS_DEFINE_TIMELINE()                                                                       \
  TS_EXPORT int ts_timeline_read(void* out, int capacity, int reset) {                             \
    unsigned n = 0;                                                                                \
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;                                         \
    if (cudaMemcpyFromSymbol(&n, g_timeline_count, sizeof(n)) != cudaSuccess) return -1;           \
    if (n > TIMELINE_CAPACITY) n = TIMELINE_CAPACITY;                                              \
    if ((int)n > capacity) n = capacity;                                                           \
    if (n && cudaMemcpyFromSymbol(out, g_timeline, n * sizeof(TimelineRecord)) != cudaSuccess) return -1; \
    const unsigned zero = 0;                                                                       \
    if (reset && cudaMemcpyToSymbol(g_timeline_count, &zero, sizeof(zero)) != cudaSuccess) return -1;     \
    return (int)n;                                                                                 \
  }
#else
__device__ __forceinline__ void timeline_mark(int) {}
__device__ __forceinline__ void timeline_mark_thread(int, int) {}
#define TS_DEFINE_TIMELINE()
#endif

// ---------------------------------------------------------------- status words
// Kernels never trap.  A kernel that gives up on a bounded wait, and the index check of a step
// (ts_sanitize_step / ts_sanitize_group in elementwise.cu) when it meets an index outside its
// buffer, store a code into a few words of pinned host memory that the engine reads after it has
// synchronised for a step's tokens anyway.  Word 0: a wait ran out.  Word 1: an index was out of
// range (the code says which buffer).  ts_set_status_words() hands the words' address to the
// library once per device.
static __device__ int* g_status_words = nullptr;
enum { TS_STATUS_WAIT = 0, TS_STATUS_BOUNDS = 1 };
enum { TS_BAD_TOKEN_ID = 1, TS_BAD_CACHE_SLOT = 2, TS_BAD_PAGE = 3, TS_BAD_POSITION = 4, TS_BAD_ROW = 5,
       TS_BAD_STATE_SLOT = 6, TS_BAD_REQUEST = 7 };
__device__ __forceinline__ void ts_raise_status(int word, int code) {
  int* w = g_status_words;
  if (w != nullptr) {
    *reinterpret_cast<volatile int*>(w + word) = code;
    __threadfence_system();
  }
}

#define TS_DEFINE_LAST_ERROR() \
  TS_DEFINE_TIMELINE()         \
  TS_EXPORT const char* ts_last_error() { return ts_error_message; }                                  \
  TS_EXPORT int ts_set_status_words(int* words) {                                                     \
    return cudaMemcpyToSymbol(g_status_words, &words, sizeof(words)) == cudaSuccess ? 0 : 1;          \
  }

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of this package is launched so that it may start while its predecessor in the
// stream still runs.  A kernel calls pdl_trigger() at its top (its successor may be launched as
// soon as all of this kernel's blocks have started) and pdl_wait() before it reads anything a
// predecessor wrote and before it writes global memory at all; pdl_wait() returns when the
// predecessor has completed and its writes are visible.  What a kernel does before pdl_wait()
// (set-up, fetching weights) overlaps the predecessor.  Set TINYSERVE_PDL=0 to launch plainly.
__device__ __forceinline__ void pdl_trigger() {
  timeline_mark(0);
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  timeline_mark(1);
}

static inline bool ts_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("TINYSERVE_PDL");
    enabled = (v && v[0] == '0') ? 0 : 1;
  }
  return enabled != 0;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t ts_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ts_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// the same with thread-block clusters (the grid a multiple of the cluster in every dimension)
template <typename... KArgs, typename... Args>
static inline cudaError_t ts_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ts_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// distributed shared memory of a cluster: rank, barrier, and a load from a peer block's copy of
// a shared variable
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float cluster_load_f32(const float* own_shared, uint32_t rank) {
  uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(own_shared)), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

#define TS_LAUNCH(name, kernel, grid, block, smem, stream, ...)                          \
  do {                                                                                   \
    cudaError_t e_ = ts_launch(kernel, grid, block, smem, stream, __VA_ARGS__);          \
    if (e_ != cudaSuccess) return ts_fail("%s: %s", name, cudaGetErrorString(e_));       \
  } while (0)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// gated feed-forward: act(gate) * up
enum { ACT_SILU = 0, ACT_GELU_TANH = 1 };
__device__ __forceinline__ float activate(float g, int act) {
  if (act == ACT_SILU) return g / (1.f + expf(-g));
  const float c = 0.7978845608028654f;
  return 0.5f * g * (1.f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// a weight vector that is either float or bfloat16, chosen at run time
struct VecParam {
  const void* ptr;
  int is_f32;
  __device__ __forceinline__ float operator[](int i) const {
    return is_f32 ? static_cast<const float*>(ptr)[i]
                  : __bfloat162float(static_cast<const __nv_bfloat16*>(ptr)[i]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Split-K partial tiles of a product [M, N] as gemm_tcgen05.cu leaves them when it is asked for
// partials only: [split][token tile][row tile][token in tile][row in tile (128)], float.  A
// consumer kernel adds the splits while it loads, in split order, so the sum is the same every run.
struct PartialSrc {
  const float* base;      // null: there are no partials, the consumer reads its ordinary input
  int splits, n_tiles, t_tiles, tile_t;
  __device__ __forceinline__ size_t offset(int s, int m, int n) const {
    const int tile = (m / tile_t) * n_tiles + (n >> 7);
    return (((size_t)s * (n_tiles * t_tiles) + tile) * tile_t + m % tile_t) * 128 + (n & 127);
  }
  __device__ __forceinline__ float load1(int m, int n) const {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += __ldcg(base + offset(s, m, n));
    return v;
  }
  __device__ __forceinline__ float2 load2(int m, int n) const {      // n even
    float2 v = make_float2(0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float2 q = __ldcg(reinterpret_cast<const float2*>(base + offset(s, m, n)));
      v.x += q.x; v.y += q.y;
    }
    return v;
  }
  __device__ __forceinline__ void load4(int m, int n, float (&v)[4]) const {   // n a multiple of 4
    v[0] = v[1] = v[2] = v[3] = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(base + offset(s, m, n)));
      v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
    }
  }
};

// sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
