// Paged, variable-length, causal grouped-query attention with 32-bit arithmetic on the
// CUDA cores, for one head size per build (-DTS_HEAD_DIM=...).  It serves the true 32-bit
// path for prefill and decode, and bfloat16 storage for head sizes that the tensor-core
// kernels do not take.
//
// Behaviour follows serve.py:639-688: request b's queries are rows cu_q[b]..cu_q[b+1] of
// q; query i stands at position kv_len - q_len + i; key j is visible iff j <= position
// (and, with a window W > 0, j > position - W); query head h reads KV head h / (H / Hkv);
// keys are found through the request's block table.  Online softmax as
// tinykernels.py:386-413, but with every product and sum in 32-bit.
//
// A block handles 32 rows = (query, head of one KV group) pairs, so that one pass over the
// keys serves the whole group, and optionally one of `num_splits` ranges of the keys
// (tinykernels.py:865-889); ts_attention_combine merges the ranges (tinykernels.py:800-853).
#include "common.cuh"

#ifndef TS_HEAD_DIM
#error "compile with -DTS_HEAD_DIM=<head size, a multiple of 16>"
#endif

TS_DEFINE_LAST_ERROR()

namespace {

constexpr int D = TS_HEAD_DIM;
constexpr int BM = 32;       // rows of a block
constexpr int BN = 32;       // keys of a tile
constexpr int WARPS = 4;
constexpr int RPW = BM / WARPS;            // rows of a warp
constexpr int DC = (D + 31) / 32;          // output columns of a lane
constexpr int KS = D + 1;                  // row stride of the key tile in shared memory
static_assert(D % 16 == 0 && D >= 16 && D <= 512, "head size must be a multiple of 16 up to 512");

struct AttnParams {
  const void* q;            // [T, H, D]
  void* out;                // [T, H, D]
  const void* k_cache;      // [pages, Hkv, page_size, D]
  const void* v_cache;
  const int* block_table;   // [B, max_blocks]
  const int* cu_q;          // [B + 1]
  const int* kv_lens;       // [B]
  float* part_o;            // [T, H, splits, D] (num_splits > 1)
  float* part_ml;           // [T, H, splits, 2]
  int H, Hkv, page_size, max_blocks;
  int heads_per_tile, queries_per_tile, head_tiles;
  int num_splits, window;
  float scale;
};

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_row_chunk(const T* p, float* dst);
template <>
__device__ __forceinline__ void load_row_chunk<float>(const float* p, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load_row_chunk<__nv_bfloat16>(const __nv_bfloat16* p, float* dst) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __low2float(h[i]);
    dst[2 * i + 1] = __high2float(h[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(AttnParams p) {
  extern __shared__ float smem[];
  float* Qs = smem;                    // [BM][D]
  float* Ks = Qs + BM * D;             // [BN][KS]
  float* Vs = Ks + BN * KS;            // [BN][D]
  float* Ps = Vs + BN * D;             // [BM][BN]

  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.z / p.num_splits, split = blockIdx.z % p.num_splits;
  const int kvh = blockIdx.y / p.head_tiles, head_tile = blockIdx.y % p.head_tiles;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = blockIdx.x * p.queries_per_tile;
  if (q0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int G = p.H / p.Hkv, GT = p.heads_per_tile;
  const int g0 = head_tile * GT;
  const int nq = min(p.queries_per_tile, q_len - q0);
  const int ng = min(GT, G - g0);
  const int n_valid = p.queries_per_tile > 1 ? nq * GT : ng;   // valid rows are a prefix
  const int pos0 = kv_len - q_len + q0;                        // position of the tile's first query
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q = static_cast<const T*>(p.q);
  const T* kc = static_cast<const T*>(p.k_cache);
  const T* vc = static_cast<const T*>(p.v_cache);

  // queries of the tile -> shared memory
  for (int i = threadIdx.x; i < BM * D; i += WARPS * 32) {
    const int r = i / D, d = i % D;
    float v = 0.f;
    if (r < n_valid) {
      const int qi = r / GT, g = r % GT;
      v = to_f32<T>(q[((size_t)(q_begin + q0 + qi) * p.H + kvh * G + g0 + g) * D + d]);
    }
    Qs[i] = v;
  }

  // key range of this tile and of this split
  const int j_hi = min(kv_len, pos0 + nq);
  const int j_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_tile = j_lo / BN;
  const int total_tiles = (j_hi + BN - 1) / BN - first_tile;
  const int per_split = (total_tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(first_tile + total_tiles, tile_begin + per_split);

  float m[RPW], l[RPW], acc[RPW][DC];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[i][c] = 0.f;
  }

  constexpr int VN = Vec16<T>::N, CHUNKS = D / VN;
  const int* bt = p.block_table + (size_t)b * p.max_blocks;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int j0 = tile * BN;
    __syncthreads();   // the previous tile's keys and values are no longer read
    for (int i = threadIdx.x; i < BN * CHUNKS; i += WARPS * 32) {
      const int key = i / CHUNKS, c = (i % CHUNKS) * VN;
      const int j = j0 + key;
      float kv[VN], vv[VN];
      if (j >= j_lo && j < j_hi) {
        const size_t page = bt[j / p.page_size];
        const size_t off = ((page * p.Hkv + kvh) * p.page_size + j % p.page_size) * D + c;
        load_row_chunk<T>(kc + off, kv);
        load_row_chunk<T>(vc + off, vv);
      } else {
#pragma unroll
        for (int e = 0; e < VN; ++e) kv[e] = vv[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        Ks[key * KS + c + e] = kv[e];
        Vs[key * D + c + e] = vv[e];
      }
    }
    __syncthreads();

    // scores of this warp's rows against key `lane`
    const int j = j0 + lane;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const int r = warp + WARPS * i;
      if (r >= n_valid) break;
      const float* qr = Qs + r * D;
      const float* kr = Ks + lane * KS;
      float s = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      s *= p.scale;
      const int pos = pos0 + (p.queries_per_tile > 1 ? r / GT : 0);
      const bool visible = j <= pos && j < j_hi && (p.window <= 0 || j > pos - p.window);
      s = visible ? s : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(s));
      const float prob = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float alpha = (m[i] == -INFINITY) ? 0.f : expf(m[i] - m_new);
      l[i] = l[i] * alpha + warp_sum(prob);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[i][c] *= alpha;
      Ps[r * BN + lane] = prob;
    }
    __syncwarp();
    // acc += P * V
    for (int key = 0; key < BN; ++key) {
      float v[DC];
#pragma unroll
      for (int c = 0; c < DC; ++c) v[c] = (D % 32 == 0 || lane + 32 * c < D) ? Vs[key * D + lane + 32 * c] : 0.f;
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const int r = warp + WARPS * i;
        if (r >= n_valid) break;
        const float pr = Ps[r * BN + key];
#pragma unroll
        for (int c = 0; c < DC; ++c) acc[i][c] = fmaf(pr, v[c], acc[i][c]);
      }
    }
    __syncwarp();
  }

  // results
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = warp + WARPS * i;
    if (r >= n_valid) break;
    const int qi = p.queries_per_tile > 1 ? r / GT : 0, g = r % GT;
    const size_t row = (size_t)(q_begin + q0 + qi) * p.H + kvh * G + g0 + g;
    if (p.num_splits == 1) {
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
      T* o = static_cast<T*>(p.out) + row * D;
#pragma unroll
      for (int c = 0; c < DC; ++c)
        if (D % 32 == 0 || lane + 32 * c < D) o[lane + 32 * c] = from_f32<T>(acc[i][c] * inv);
    } else {
      float* o = p.part_o + (row * p.num_splits + split) * D;
#pragma unroll
      for (int c = 0; c < DC; ++c)
        if (D % 32 == 0 || lane + 32 * c < D) o[lane + 32 * c] = acc[i][c];
      if (lane == 0) {
        p.part_ml[(row * p.num_splits + split) * 2] = m[i];
        p.part_ml[(row * p.num_splits + split) * 2 + 1] = l[i];
      }
    }
  }
}

// out[row] = sum_s exp(m_s - m) o_s / sum_s exp(m_s - m) l_s over the splits of a row
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, T* __restrict__ out,
                                         int num_splits) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = part_ml + row * num_splits * 2;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, ml[2 * s]);
  float denom = 0.f;
  for (int s = 0; s < num_splits; ++s)
    denom += (ml[2 * s] == -INFINITY) ? 0.f : expf(ml[2 * s] - m) * ml[2 * s + 1];
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = (ml[2 * s] == -INFINITY) ? 0.f : expf(ml[2 * s] - m);
      v = fmaf(w, part_o[(row * num_splits + s) * D + d], v);
    }
    out[row * D + d] = from_f32<T>(v * inv);
  }
}

size_t smem_bytes() { return sizeof(float) * (BM * D + BN * KS + BN * D + BM * BN); }

}  // namespace

TS_EXPORT int ts_attention_head_dim() { return D; }

// Scratch for num_splits > 1: part_o holds T*H*splits*D floats, part_ml T*H*splits*2.
TS_EXPORT int ts_paged_attention(int dtype, const void* q, void* out, const void* k_cache,
                                 const void* v_cache, const int* block_table, const int* cu_q,
                                 const int* kv_lens, int num_tokens, int num_requests,
                                 int max_q_len, int H, int Hkv, int page_size, int max_blocks,
                                 float scale, int window, int num_splits, float* part_o,
                                 float* part_ml, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && num_requests > 0 && max_q_len > 0, "paged_attention: empty batch");
  TS_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0, "paged_attention: %d heads over %d KV heads", H, Hkv);
  TS_REQUIRE(page_size > 0 && max_blocks > 0, "paged_attention: bad page geometry");
  TS_REQUIRE(num_splits >= 1 && num_splits <= 64, "paged_attention: num_splits %d out of range", num_splits);
  TS_REQUIRE(num_splits == 1 || (part_o && part_ml), "paged_attention: splits without scratch");
  TS_REQUIRE(dtype == TS_F32 || dtype == TS_BF16, "paged_attention: unknown dtype %d", dtype);
  AttnParams p;
  p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache;
  p.block_table = block_table; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.part_o = part_o; p.part_ml = part_ml;
  p.H = H; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks;
  const int G = H / Hkv;
  p.heads_per_tile = G < BM ? G : BM;
  p.queries_per_tile = G < BM ? BM / G : 1;
  p.head_tiles = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  p.num_splits = num_splits; p.window = window; p.scale = scale;
  const long long gz = (long long)num_requests * num_splits;
  const long long gy = (long long)Hkv * p.head_tiles;
  TS_REQUIRE(gz <= 65535 && gy <= 65535, "paged_attention: grid too large (%lld requests*splits, %lld head tiles)", gz, gy);
  dim3 grid((max_q_len + p.queries_per_tile - 1) / p.queries_per_tile, (unsigned)gy, (unsigned)gz);
  const size_t smem = smem_bytes();
  cudaError_t e;
  if (dtype == TS_F32) {
    e = cudaFuncSetAttribute(paged_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("paged_attention: %s", cudaGetErrorString(e));
    TS_LAUNCH("paged_attention", paged_attention_kernel<float>, grid, WARPS * 32, smem, stream, p);
  } else {
    e = cudaFuncSetAttribute(paged_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("paged_attention: %s", cudaGetErrorString(e));
    TS_LAUNCH("paged_attention", paged_attention_kernel<__nv_bfloat16>, grid, WARPS * 32, smem, stream, p);
  }
  if (num_splits > 1) {
    const int threads = D >= 128 ? 128 : (D >= 64 ? 64 : 32);
    if (dtype == TS_F32)
      TS_LAUNCH("attention_combine", attention_combine_kernel<float>, num_tokens * H, threads, 0, stream, (const float*)part_o, (const float*)part_ml, (float*)out, num_splits);
    else
      TS_LAUNCH("attention_combine", attention_combine_kernel<__nv_bfloat16>, num_tokens * H, threads, 0, stream, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, num_splits);
  }
  return 0;
}

// ------------------------------------------------------------------ no-allocation entry point
// See attention_static_scratch.h: the same kernels, with the split scratch in a fixed array of
// the library image instead of caller memory.  Host code may not use the array's name as a
// pointer (it is a host-side stand-in for the symbol); its device address comes from
// cudaGetSymbolAddress, once per device, and is what the kernels are given.
#include "attention_static_scratch.h"

static __device__ __align__(256) float ts_static_scratch[TS_STATIC_SCRATCH_FLOATS];

#include <mutex>

namespace {
constexpr int MAX_DEVICES = 64;
float* static_scratch_address[MAX_DEVICES] = {nullptr};
std::mutex static_scratch_mutex;       // guards the table above (first calls from several threads)
}  // namespace

TS_EXPORT int ts_paged_attention_static_scratch(
    int dtype, const void* q, void* out, const void* k_cache, const void* v_cache,
    const int* block_table, const int* cu_q, const int* kv_lens, int num_tokens, int num_requests,
    int max_q_len, int H, int Hkv, int page_size, int max_blocks, float scale, int window,
    int num_splits, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && num_splits >= 1, "paged_attention_static_scratch: empty batch");
  const long long rows = (long long)num_tokens * H * num_splits;
  // one key range needs no scratch at all: the kernel writes its output directly
  const long long need = num_splits > 1 ? rows * (D + 2) : 0;
  TS_REQUIRE(need <= (long long)TS_STATIC_SCRATCH_FLOATS,
             "paged_attention_static_scratch: %d tokens x %d heads x %d splits need %lld floats of "
             "scratch, the static array holds %d",
             num_tokens, H, num_splits, need, (int)TS_STATIC_SCRATCH_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return ts_fail("paged_attention_static_scratch: %s", cudaGetErrorString(e));
  TS_REQUIRE(device >= 0 && device < MAX_DEVICES, "paged_attention_static_scratch: device %d out of range", device);
  float* part_o = nullptr;
  {
    std::lock_guard<std::mutex> lock(static_scratch_mutex);
    if (static_scratch_address[device] == nullptr) {
      float* address = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), ts_static_scratch);
      if (e != cudaSuccess || address == nullptr)
        return ts_fail("paged_attention_static_scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      static_scratch_address[device] = address;
    }
    part_o = static_scratch_address[device];
  }
  float* part_ml = part_o + rows * D;
  return ts_paged_attention(dtype, q, out, k_cache, v_cache, block_table, cu_q, kv_lens, num_tokens,
                            num_requests, max_q_len, H, Hkv, page_size, max_blocks, scale, window,
                            num_splits, part_o, part_ml, stream);
}
