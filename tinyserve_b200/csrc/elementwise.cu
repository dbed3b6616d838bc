// Memory-bound kernels of the forward pass: embedding lookup, (residual add +) RMSNorm,
// gated activation, and the fused per-head norm + rotary encoding + cache write.
// All arithmetic is 32-bit; T is the storage type of activations (float or bfloat16).
//
// Reference behaviour: tinykernels.py:26-61 (residual add + RMSNorm), 107-218 (q/k norm,
// RoPE, cache write in one kernel), 277-297 (SiLU * up); serve.py:1239 (embedding).
#include "common.cuh"

TS_DEFINE_LAST_ERROR()

// ------------------------------------------------------------------ embedding
// An id < 0 stands for a token that is still on the device: -1 - slot names the state slot of the
// request, whose last sampled token the sampler left in slot_tokens[slot].
template <typename T>
__global__ void embed_lookup_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int n, int vocab,
                                    const int* __restrict__ slot_tokens) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && slot_tokens) id = slot_tokens[-1 - id];
  float* dst = out + (size_t)t * n;
  if (id < 0 || id >= vocab) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

TS_EXPORT int ts_embed_lookup(int dtype, const void* table, const int* ids, float* out,
                              int num_tokens, int n, int vocab, const int* slot_tokens,
                              cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && n > 0 && vocab > 0, "embed_lookup: empty input");
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype == TS_F32)
    TS_LAUNCH("embed_lookup", embed_lookup_kernel<float>, num_tokens, threads, 0, stream, (const float*)table, ids, out, n, vocab, slot_tokens);
  else if (dtype == TS_BF16)
    TS_LAUNCH("embed_lookup", embed_lookup_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, n, vocab, slot_tokens);
  else
    return ts_fail("embed_lookup: unknown dtype %d", dtype);
  return 0;
}

// ------------------------------------------------------------------ block tables on the device
// Every state slot keeps its request's block-table row on the device ("resident", [groups][slots +
// 1][max_blocks]); a step uploads only the entries that changed (pairs of flat index and page) and
// these two kernels bring the rows of the step's requests into the [groups][requests][max_blocks]
// tables that the attention kernels index by request.  The number of pairs is read from device
// memory, so that a captured graph serves any step.
__global__ void block_table_scatter_kernel(int* __restrict__ resident, long long resident_size,
                                           const int* __restrict__ pairs, const int* __restrict__ num_pairs,
                                           int capacity) {
  pdl_trigger();
  pdl_wait();
  const int n = min(*num_pairs, capacity);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int at = pairs[2 * i];
    if (at >= 0 && at < resident_size) resident[at] = pairs[2 * i + 1];
  }
}

__global__ void block_table_gather_kernel(const int* __restrict__ resident, int* __restrict__ step_tables,
                                          const int* __restrict__ state_slots, int num_slots, int max_requests,
                                          int max_blocks) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, g = blockIdx.y;
  int slot = state_slots[b];
  if (slot < 0 || slot > num_slots) slot = num_slots;          // the spare row: all null pages
  const int* src = resident + ((size_t)g * (num_slots + 1) + slot) * max_blocks;
  int* dst = step_tables + ((size_t)g * max_requests + b) * max_blocks;
  for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) dst[i] = src[i];
}

// resident [groups][num_slots + 1][max_blocks]; pairs [capacity][2] and num_pairs [1] on the device;
// step_tables [groups][max_requests][max_blocks]; state_slots [num_requests].
TS_EXPORT int ts_block_tables_step(int* resident, const int* pairs, const int* num_pairs, int capacity,
                                   int* step_tables, const int* state_slots, int num_requests, int max_requests,
                                   int num_slots, int max_blocks, int groups, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && num_requests <= max_requests && groups > 0 && max_blocks > 0 && capacity >= 0,
             "block_tables_step: empty step");
  const long long size = (long long)groups * (num_slots + 1) * max_blocks;
  TS_LAUNCH("block_table_scatter", block_table_scatter_kernel, 8, 256, 0, stream, resident, size, pairs, num_pairs,
            capacity);
  TS_LAUNCH("block_table_gather", block_table_gather_kernel, dim3(num_requests, groups), 128, 0, stream,
            (const int*)resident, step_tables, state_slots, num_slots, max_requests, max_blocks);
  return 0;
}

// ------------------------------------------------------------------ index check of a step
// The debug pass that stands where a memory checker would: before a step's kernels run, one small
// kernel looks at every index the step brings.  An index outside its buffer is replaced by a
// harmless one (token 0, position 0, row 0, "no cache slot", the null page, an empty request), so
// that no later kernel reads or writes out of bounds, and its kind is stored in the status words
// (common.cuh), which the engine turns into an error.  Off in serving; tests switch it on.
__global__ void sanitize_step_kernel(int* token_ids, int T, int vocab, int* slot_tokens, int num_state_slots,
                                     int* positions, int num_positions, int* logit_rows, int W, int* cu_q,
                                     int* kv_lens, int B, int max_kv_len, int* state_slots) {
  pdl_trigger();
  pdl_wait();
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const int id = token_ids[t];
    if (id >= vocab) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_TOKEN_ID);
      token_ids[t] = 0;
    } else if (id < 0) {
      const int slot = -1 - id;
      if (slot_tokens == nullptr || slot >= num_state_slots) {
        ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_STATE_SLOT);
        token_ids[t] = 0;
      } else if (slot_tokens[slot] < 0 || slot_tokens[slot] >= vocab) {
        ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_TOKEN_ID);
        slot_tokens[slot] = 0;
      }
    }
    if (positions[t] < 0 || positions[t] >= num_positions) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_POSITION);
      positions[t] = 0;
    }
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    if (logit_rows[i] < 0 || logit_rows[i] >= T) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_ROW);
      logit_rows[i] = 0;
    }
  __shared__ int bad_requests;
  if (threadIdx.x == 0) bad_requests = cu_q[0] != 0 || cu_q[B] > T;
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int n = cu_q[b + 1] - cu_q[b];
    if (n < 0) atomicOr(&bad_requests, 1);
    if (kv_lens[b] < 0 || kv_lens[b] > max_kv_len || (n > 0 && kv_lens[b] < n)) atomicOr(&bad_requests, 1);
    if (state_slots[b] < 0 || state_slots[b] >= num_state_slots) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_STATE_SLOT);
      state_slots[b] = 0;
    }
  }
  __syncthreads();
  if (bad_requests) {
    // the requests' extents do not fit the batch: nobody brings a token, nobody holds a key
    if (threadIdx.x == 0) ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_REQUEST);
    for (int b = threadIdx.x; b <= B; b += blockDim.x) {
      cu_q[b] = 0;
      if (b < B) kv_lens[b] = 0;
    }
  }
}

__global__ void sanitize_group_kernel(int* slot_mapping, int T, long long total_slots, int* block_table, int B,
                                      int max_blocks, int row_stride, int num_pages) {
  pdl_trigger();
  pdl_wait();
  for (int t = threadIdx.x; t < T; t += blockDim.x)
    if (slot_mapping[t] < -1 || slot_mapping[t] >= total_slots) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_CACHE_SLOT);
      slot_mapping[t] = -1;
    }
  for (int i = threadIdx.x; i < B * max_blocks; i += blockDim.x) {
    int* entry = block_table + (size_t)(i / max_blocks) * row_stride + i % max_blocks;
    if (*entry < 0 || *entry >= num_pages) {
      ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_PAGE);
      *entry = 0;
    }
  }
}

// token_ids, positions [T]; logit_rows [W]; cu_q [B + 1]; kv_lens, state_slots [B]; slot_tokens
// [num_state_slots] or null.  All are read and, where out of range, rewritten in place.
TS_EXPORT int ts_sanitize_step(int* token_ids, int T, int vocab, int* slot_tokens, int num_state_slots, int* positions,
                               int num_positions, int* logit_rows, int W, int* cu_q, int* kv_lens, int B,
                               int max_kv_len, int* state_slots, cudaStream_t stream) {
  TS_REQUIRE(T > 0 && B > 0 && W >= 0 && vocab > 0 && num_positions > 0, "sanitize_step: empty step");
  TS_LAUNCH("sanitize_step", sanitize_step_kernel, 1, 256, 0, stream, token_ids, T, vocab, slot_tokens, num_state_slots,
            positions, num_positions, logit_rows, W, cu_q, kv_lens, B, max_kv_len, state_slots);
  return 0;
}

// slot_mapping [T] (page * page_size + slot, -1: none) of a pool of total_slots slots; block_table
// [B, max_blocks] with rows row_stride apart, entries below num_pages.
TS_EXPORT int ts_sanitize_group(int* slot_mapping, int T, long long total_slots, int* block_table, int B, int max_blocks,
                                int row_stride, int num_pages, cudaStream_t stream) {
  TS_REQUIRE(T > 0 && B > 0 && max_blocks > 0 && num_pages > 0, "sanitize_group: empty step");
  TS_LAUNCH("sanitize_group", sanitize_group_kernel, 1, 256, 0, stream, slot_mapping, T, total_slots, block_table, B,
            max_blocks, row_stride, num_pages);
  return 0;
}

// ------------------------------------------------------------------ residual add + RMSNorm
// One block per output row.  v = residual[r] + x[r] (x may be null), residual[r] = v when
// `write_residual`, out[i] = v * rsqrt(mean(v^2) + eps) * w.  With `rows`, output row i reads
// input row rows[i].  The order of the sum depends on n and the block size only.
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, float* __restrict__ residual,
                                   VecParam w, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int n, int write_residual, PartialSrc ps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  const T* xr = x ? x + r * n : nullptr;
  float* rr = residual + r * n;
  float acc = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float v = rr[c];
    if (ps.base) v += ps.load1((int)r, c);
    else if (xr) v += to_f32<T>(xr[c]);
    acc += v * v;
  }
  const float total = block_sum(acc, scratch);
  const float rstd = rsqrtf(total / (float)n + eps);
  T* o = out + (size_t)i * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float v = rr[c];
    if (ps.base) v += ps.load1((int)r, c);
    else if (xr) v += to_f32<T>(xr[c]);
    if (write_residual) rr[c] = v;
    o[c] = from_f32<T>(v * rstd * w[c]);
  }
}


// The same, for rows whose length is a multiple of 4 and at most 4 * 4 * blockDim: every thread
// keeps its elements in registers between the sum of squares and the output, and moves 16 bytes
// at a time.
template <typename T> struct Quad;
template <> struct Quad<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Quad<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<const uint32_t*>(&a);
    q.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = q;
  }
};

// MAX_THREADS / MIN_BLOCKS bound the registers: with many rows (prefill) the kernel lives on the
// number of rows in flight per SM, and four element groups per thread would otherwise leave room
// for two blocks only.
template <typename T, int ITEMS, int MAX_THREADS = 1024, int MIN_BLOCKS = 1>
__global__ void __launch_bounds__(MAX_THREADS, MIN_BLOCKS) add_rmsnorm_vec_kernel(const T* __restrict__ x, float* __restrict__ residual, VecParam w,
                                       float eps, T* __restrict__ out, const int* __restrict__ rows,
                                       int n, int write_residual, PartialSrc ps) {
  __shared__ float scratch[33];
  pdl_trigger();
  // the weights are constants: fetch them while the predecessor still runs (few rows: the
  // shortest chain), or where they are used (many rows: fewer registers, more rows in flight)
  constexpr bool PRELOAD = MIN_BLOCKS == 1;
  float wv[PRELOAD ? ITEMS : 1][4];
  if (PRELOAD) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int c = (threadIdx.x + it * blockDim.x) * 4;
      if (c < n) {
        if (w.is_f32) Quad<float>::load(static_cast<const float*>(w.ptr) + c, wv[it]);
        else Quad<__nv_bfloat16>::load(static_cast<const __nv_bfloat16*>(w.ptr) + c, wv[it]);
      }
    }
  }
  pdl_wait();
  const int i = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  float v[ITEMS][4];
  float acc = 0.f;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int c = (threadIdx.x + it * blockDim.x) * 4;
    if (c < n) {
      Quad<float>::load(residual + r * n + c, v[it]);
      if (ps.base || x) {
        float xv[4];
        if (ps.base) ps.load4((int)r, c, xv);
        else Quad<T>::load(x + r * n + c, xv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[it][e] += xv[e];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) acc += v[it][e] * v[it][e];
    }
  }
  const float rstd = rsqrtf(block_sum(acc, scratch) / (float)n + eps);
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int c = (threadIdx.x + it * blockDim.x) * 4;
    if (c < n) {
      if (write_residual) Quad<float>::store(residual + r * n + c, v[it]);
      if (!PRELOAD) {
        if (w.is_f32) Quad<float>::load(static_cast<const float*>(w.ptr) + c, wv[0]);
        else Quad<__nv_bfloat16>::load(static_cast<const __nv_bfloat16*>(w.ptr) + c, wv[0]);
      }
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = v[it][e] * rstd * wv[PRELOAD ? it : 0][e];
      Quad<T>::store(out + (size_t)i * n + c, o);
    }
  }
}

// Few rows (decode): a row is spread over a cluster of NORM_CLUSTER blocks, so that its partial
// sums of a split-K product, which are many times the row itself, come in through that many SMs.
// Each block adds up the squares of its columns, the blocks read one another's sums from
// distributed shared memory in rank order (every block gets the same total, the same every run)
// and each normalises its own columns.  Blocks of a cluster are (rank, row).
constexpr int NORM_CLUSTER = 8;
constexpr int PARTIAL_BATCH = 8;      // loads of partial sums in flight per thread

template <typename T>
__global__ void add_rmsnorm_cluster_kernel(const T* __restrict__ x, float* __restrict__ residual, VecParam w,
                                           float eps, T* __restrict__ out, const int* __restrict__ rows,
                                           int n, int quads_per_block, int write_residual, PartialSrc ps) {
  __shared__ float scratch[33];
  __shared__ float cluster_part;
  pdl_trigger();
  const uint32_t rank = cluster_rank();
  const int c = ((int)rank * quads_per_block + (int)threadIdx.x) * 4;
  const bool active = (int)threadIdx.x < quads_per_block && c < n;
  float wv[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {      // the weights are constants: fetch them while the predecessor still runs
    if (w.is_f32) Quad<float>::load(static_cast<const float*>(w.ptr) + c, wv);
    else Quad<__nv_bfloat16>::load(static_cast<const __nv_bfloat16*>(w.ptr) + c, wv);
  }
  pdl_wait();
  const int i = blockIdx.y;
  const size_t r = rows ? (size_t)rows[i] : (size_t)i;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  float acc = 0.f;
  if (active) {
    Quad<float>::load(residual + r * n + c, v);
    if (ps.base) {
      // all loads of a batch are issued before the first is used; the sum runs in split order
      float xs[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < ps.splits; s0 += PARTIAL_BATCH) {
        float4 q[PARTIAL_BATCH];
#pragma unroll
        for (int s = 0; s < PARTIAL_BATCH; ++s)
          if (s0 + s < ps.splits) q[s] = __ldcg(reinterpret_cast<const float4*>(ps.base + ps.offset(s0 + s, (int)r, c)));
#pragma unroll
        for (int s = 0; s < PARTIAL_BATCH; ++s)
          if (s0 + s < ps.splits) { xs[0] += q[s].x; xs[1] += q[s].y; xs[2] += q[s].z; xs[3] += q[s].w; }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] += xs[e];
    } else if (x) {
      float xv[4];
      Quad<T>::load(x + r * n + c, xv);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] += xv[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) acc += v[e] * v[e];
  }
  const float mine = block_sum(acc, scratch);
  if (threadIdx.x == 0) cluster_part = mine;
  cluster_arrive();
  cluster_wait();
  float total = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_CLUSTER; ++k) total += cluster_load_f32(&cluster_part, k);
  cluster_arrive();        // this block has read its peers; it may not leave before they have read it
  const float rstd = rsqrtf(total / (float)n + eps);
  if (active) {
    if (write_residual) Quad<float>::store(residual + r * n + c, v);
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = v[e] * rstd * wv[e];
    Quad<T>::store(out + (size_t)i * n + c, o);
  }
  cluster_wait();
}

template <typename T>
int launch_add_rmsnorm(const void* x, float* residual, VecParam w, float eps, void* out, const int* rows,
                       int num_out_rows, int n, int write_residual, PartialSrc ps, cudaStream_t stream) {
  const bool aligned = n % 4 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) |
                                      reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w.ptr)) % 16 == 0;
  const T* xp = static_cast<const T*>(x);
  T* op = static_cast<T*>(out);
  if (aligned && num_out_rows <= 32 && n >= 1024 && n <= NORM_CLUSTER * 4 * 1024) {
    const int quads_per_block = (n / 4 + NORM_CLUSTER - 1) / NORM_CLUSTER;
    const int threads = (quads_per_block + 31) / 32 * 32;
    cudaError_t e = ts_launch_cluster(add_rmsnorm_cluster_kernel<T>, dim3(NORM_CLUSTER, num_out_rows), dim3(threads), 0,
                                      stream, dim3(NORM_CLUSTER), xp, residual, w, eps, op, rows, n, quads_per_block,
                                      write_residual, ps);
    if (e != cudaSuccess) return ts_fail("add_rmsnorm: %s", cudaGetErrorString(e));
    return 0;
  }
  if (aligned && n <= 4 * 4 * 1024) {
    const int quads = n / 4;
    // few rows (decode): one element group per thread, the shortest chain; many rows (prefill):
    // smaller blocks with four groups per thread, more rows in flight per SM
    int items = quads <= 1024 ? 1 : (quads <= 2048 ? 2 : 4);
    if (num_out_rows >= 512 && quads >= 256) items = 4;
    int threads = ((quads + items - 1) / items + 31) / 32 * 32;
    if (items == 1) TS_LAUNCH("add_rmsnorm", (add_rmsnorm_vec_kernel<T, 1>), num_out_rows, threads, 0, stream, xp, residual, w, eps, op, rows, n, write_residual, ps);
    else if (items == 2) TS_LAUNCH("add_rmsnorm", (add_rmsnorm_vec_kernel<T, 2>), num_out_rows, threads, 0, stream, xp, residual, w, eps, op, rows, n, write_residual, ps);
    else if (threads <= 256) TS_LAUNCH("add_rmsnorm", (add_rmsnorm_vec_kernel<T, 4, 256, 4>), num_out_rows, threads, 0, stream, xp, residual, w, eps, op, rows, n, write_residual, ps);
    else TS_LAUNCH("add_rmsnorm", (add_rmsnorm_vec_kernel<T, 4>), num_out_rows, threads, 0, stream, xp, residual, w, eps, op, rows, n, write_residual, ps);
    return 0;
  }
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  TS_LAUNCH("add_rmsnorm", add_rmsnorm_kernel<T>, num_out_rows, threads, 0, stream, xp, residual, w, eps, op, rows, n, write_residual, ps);
  return 0;
}

// With `partials` (split-K partial tiles of a product [M, n], see PartialSrc) x is their sum.
TS_EXPORT int ts_add_rmsnorm(int dtype, const void* x, float* residual, const void* weight,
                             int weight_is_f32, float eps, void* out, const int* rows,
                             int num_out_rows, int n, int write_residual, const float* partials,
                             int splits, int n_tiles, int t_tiles, int tile_t, cudaStream_t stream) {
  TS_REQUIRE(num_out_rows > 0 && n > 0, "add_rmsnorm: empty input");
  TS_REQUIRE(partials == nullptr || (x == nullptr && splits > 0 && n_tiles * 128 >= n && tile_t > 0),
             "add_rmsnorm: partial tiles do not fit the row length");
  PartialSrc ps{partials, splits, n_tiles, t_tiles, tile_t};
  VecParam w{weight, weight_is_f32};
  if (dtype == TS_F32)
    return launch_add_rmsnorm<float>(x, residual, w, eps, out, rows, num_out_rows, n, write_residual, ps, stream);
  if (dtype == TS_BF16)
    return launch_add_rmsnorm<__nv_bfloat16>(x, residual, w, eps, out, rows, num_out_rows, n, write_residual, ps, stream);
  return ts_fail("add_rmsnorm: unknown dtype %d", dtype);
}

// plain RMSNorm of rows stored as T
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, VecParam w, float eps, T* __restrict__ out,
                               int n) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const T* xr = x + (size_t)blockIdx.x * n;
  float acc = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32<T>(xr[c]);
    acc += v * v;
  }
  const float rstd = rsqrtf(block_sum(acc, scratch) / (float)n + eps);
  T* o = out + (size_t)blockIdx.x * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    o[c] = from_f32<T>(to_f32<T>(xr[c]) * rstd * w[c]);
}

TS_EXPORT int ts_rmsnorm(int dtype, const void* x, const void* weight, int weight_is_f32, float eps,
                         void* out, int num_rows, int n, cudaStream_t stream) {
  TS_REQUIRE(num_rows > 0 && n > 0, "rmsnorm: empty input");
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : (n >= 64 ? 128 : 32));
  VecParam w{weight, weight_is_f32};
  if (dtype == TS_F32)
    TS_LAUNCH("rmsnorm", rmsnorm_kernel<float>, num_rows, threads, 0, stream, (const float*)x, w, eps, (float*)out, n);
  else if (dtype == TS_BF16)
    TS_LAUNCH("rmsnorm", rmsnorm_kernel<__nv_bfloat16>, num_rows, threads, 0, stream, (const __nv_bfloat16*)x, w, eps, (__nv_bfloat16*)out, n);
  else
    return ts_fail("rmsnorm: unknown dtype %d", dtype);
  return 0;
}

// ------------------------------------------------------------------ rows without their norm factor -> rows
// out[m, :] = x[m, :] * rsqrt(sum_t sumsq[t][m] / n + eps): the normalised rows of what the residual
// forms of the tcgen05 products leave (x = residual * norm_weight, sums of residual^2 per 128
// columns, `stride` floats apart)
__global__ void scale_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq, int tiles,
                                  int stride, float eps, __nv_bfloat16* __restrict__ out, int n) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  float sum = 0.f;
  for (int t = 0; t < tiles; ++t) sum += sumsq[(size_t)t * stride + m];
  const float rstd = rsqrtf(sum / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    out[(size_t)m * n + c] = __float2bfloat16_rn(__bfloat162float(x[(size_t)m * n + c]) * rstd);
}

TS_EXPORT int ts_scale_rows(const void* x, const float* sumsq, int tiles, int stride, float eps, void* out, int M,
                            int n, cudaStream_t stream) {
  TS_REQUIRE(M > 0 && M <= stride && n > 0 && tiles > 0, "scale_rows: rows with their sums of squares, at most `stride` of them");
  TS_LAUNCH("scale_rows", scale_rows_kernel, M, 256, 0, stream, (const __nv_bfloat16*)x, sumsq, tiles, stride, eps,
            (__nv_bfloat16*)out, n);
  return 0;
}

// ------------------------------------------------------------------ split-K partial tiles -> matrix
template <typename T>
__global__ void reduce_partials_kernel(PartialSrc ps, T* __restrict__ out, int N) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  for (int n = threadIdx.x; n < N; n += blockDim.x) out[(size_t)m * N + n] = from_f32<T>(ps.load1(m, n));
}

TS_EXPORT int ts_reduce_partials(int dtype, const float* partials, int splits, int n_tiles, int t_tiles,
                                 int tile_t, void* out, int M, int N, cudaStream_t stream) {
  TS_REQUIRE(partials && splits > 0 && M > 0 && N > 0 && n_tiles * 128 >= N, "reduce_partials: bad arguments");
  PartialSrc ps{partials, splits, n_tiles, t_tiles, tile_t};
  if (dtype == TS_F32) TS_LAUNCH("reduce_partials", reduce_partials_kernel<float>, M, 256, 0, stream, ps, (float*)out, N);
  else if (dtype == TS_BF16) TS_LAUNCH("reduce_partials", reduce_partials_kernel<__nv_bfloat16>, M, 256, 0, stream, ps, (__nv_bfloat16*)out, N);
  else return ts_fail("reduce_partials: unknown dtype %d", dtype);
  return 0;
}

// ------------------------------------------------------------------ gated activation
// in [rows, 2 * inter] -> out [rows, inter] = act(gate) * up.  block == 0: in = gate | up (two
// halves); block > 0: gate and up alternate in blocks of that many columns (gate columns
// [0, block), up columns [0, block), gate columns [block, 2 block), ...), the layout of a fused
// projection whose weight rows are interleaved so that one 128-row tile of the tcgen05 product
// holds matching gate and up rows.
__device__ __forceinline__ int gate_column(int c, int block) { return block ? (c / block) * 2 * block + c % block : c; }

template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ in, T* __restrict__ out, int inter,
                                        int act, int block) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= inter) return;
  const T* r = in + row * 2 * inter;
  const int g = gate_column(c, block), u = g + (block ? block : inter);
  out[row * inter + c] = from_f32<T>(activate(to_f32<T>(r[g]), act) * to_f32<T>(r[u]));
}

// 16 bytes per thread and operand, for widths that are a multiple of 16 / sizeof(T)
template <typename T>
__global__ void gated_activation_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int act,
                                            int block) {
  constexpr int V = 16 / sizeof(T);
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= inter) return;
  const T* r = in + row * 2 * inter;
  const int gc = gate_column(c, block), uc = gc + (block ? block : inter);      // block is a multiple of V
  float g[V], u[V], o[V];
#pragma unroll
  for (int h = 0; h < V / 4; ++h) {
    float a[4], b[4];
    Quad<T>::load(r + gc + 4 * h, a);
    Quad<T>::load(r + uc + 4 * h, b);
#pragma unroll
    for (int e = 0; e < 4; ++e) { g[4 * h + e] = a[e]; u[4 * h + e] = b[e]; }
  }
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = activate(g[e], act) * u[e];
#pragma unroll
  for (int h = 0; h < V / 4; ++h) {
    float a[4] = {o[4 * h], o[4 * h + 1], o[4 * h + 2], o[4 * h + 3]};
    Quad<T>::store(out + row * inter + c + 4 * h, a);
  }
}

template <typename T>
int launch_gated_activation(const void* in, void* out, int num_rows, int inter, int act, int block,
                            cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = inter % V == 0 && block % V == 0 &&
                   (reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (vec) {
    dim3 grid(num_rows, (inter / V + 255) / 256);
    TS_LAUNCH("gated_activation", gated_activation_vec_kernel<T>, grid, 256, 0, stream, (const T*)in, (T*)out, inter, act, block);
  } else {
    dim3 grid(num_rows, (inter + 255) / 256);
    TS_LAUNCH("gated_activation", gated_activation_kernel<T>, grid, 256, 0, stream, (const T*)in, (T*)out, inter, act, block);
  }
  return 0;
}

TS_EXPORT int ts_gated_activation(int dtype, const void* in, void* out, int num_rows, int inter,
                                  int act, int block, cudaStream_t stream) {
  TS_REQUIRE(num_rows > 0 && inter > 0, "gated_activation: empty input");
  TS_REQUIRE(block >= 0 && (block == 0 || inter % block == 0), "gated_activation: %d columns do not come in blocks of %d", inter, block);
  TS_REQUIRE((inter + 255) / 256 <= 65535, "gated_activation: width %d is too large", inter);
  TS_REQUIRE(act == ACT_SILU || act == ACT_GELU_TANH, "gated_activation: unknown activation %d", act);
  if (dtype == TS_F32) return launch_gated_activation<float>(in, out, num_rows, inter, act, block, stream);
  if (dtype == TS_BF16) return launch_gated_activation<__nv_bfloat16>(in, out, num_rows, inter, act, block, stream);
  return ts_fail("gated_activation: unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ q/k norm + rotary + cache write
// qkv [T, (H + 2 Hkv) * D]: q heads, k heads, v heads.  One warp per (token, head):
//   q heads: optional RMSNorm over D, rotary, stored to q_out [T, H, D];
//   k heads: the same, stored to the key page of the token's slot;
//   v heads: copied to the value page.
// A slot of -1 writes nothing.  Cache layout: [page, kv_head, slot, D].
struct RopeArgs {
  const float* cos;   // [positions, rotary_dim / 2]
  const float* sin;
  int rotary_dim;     // 0: no rotary
  int interleaved;    // pairs (2j, 2j+1) instead of (j, j + rotary_dim / 2)
};

template <typename T>
__device__ __forceinline__ void rope_one_head(int t, int head, int lane, const T* __restrict__ qkv, T* __restrict__ q_out,
                                            const int* __restrict__ positions, RopeArgs rope,
                                            VecParam qw, VecParam kw, int has_norm, float eps,
                                            int H, int Hkv, int D, T* __restrict__ k_cache,
                                            T* __restrict__ v_cache,
                                            const int* __restrict__ slot_mapping, int page_size,
                                            int heads_total, PartialSrc ps) {
  const T* src = qkv + (size_t)t * (H + 2 * Hkv) * D + (size_t)head * D;
  const int n0 = head * D;
  auto in = [&](int i) { return ps.base ? ps.load1(t, n0 + i) : to_f32<T>(src[i]); };
  T* dst;
  bool is_v = false;
  VecParam w = qw;
  if (head < H) {
    dst = q_out + ((size_t)t * H + head) * D;
  } else {
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const int kvh = head < H + Hkv ? head - H : head - H - Hkv;
    is_v = head >= H + Hkv;
    const size_t page = slot / page_size, in_page = slot % page_size;
    T* base = is_v ? v_cache : k_cache;
    dst = base + ((page * Hkv + kvh) * page_size + in_page) * D;
    w = kw;
  }
  if (is_v) {
    for (int i = lane; i < D; i += 32) dst[i] = ps.base ? from_f32<T>(in(i)) : src[i];
    return;
  }
  float rstd = 1.f;
  if (has_norm) {
    float acc = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float v = in(i);
      acc += v * v;
    }
    rstd = rsqrtf(warp_sum(acc) / (float)D + eps);
  }
  const int R = rope.rotary_dim, half = R >> 1;
  const int pos = positions[t];
  for (int j = lane; j < half; j += 32) {
    const int i0 = rope.interleaved ? 2 * j : j;
    const int i1 = rope.interleaved ? 2 * j + 1 : j + half;
    float a = in(i0), b = in(i1);
    if (has_norm) {
      a = a * rstd * w[i0];
      b = b * rstd * w[i1];
    }
    const float c = rope.cos[(size_t)pos * half + j], s = rope.sin[(size_t)pos * half + j];
    dst[i0] = from_f32<T>(a * c - b * s);
    dst[i1] = from_f32<T>(b * c + a * s);
  }
  for (int i = R + lane; i < D; i += 32) {
    float a = in(i);
    if (has_norm) a = a * rstd * w[i];
    dst[i] = from_f32<T>(a);
  }
}
// one warp per (token, head); with gridDim.y smaller than the number of head groups the warps
// walk the heads, so that many tokens need few, fatter blocks
template <typename T>
__global__ void qk_norm_rope_kvwrite_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                            const int* __restrict__ positions, RopeArgs rope,
                                            VecParam qw, VecParam kw, int has_norm, float eps,
                                            int H, int Hkv, int D, T* __restrict__ k_cache,
                                            T* __restrict__ v_cache,
                                            const int* __restrict__ slot_mapping, int page_size,
                                            int heads_total, PartialSrc ps) {
  pdl_trigger();
  pdl_wait();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int head = blockIdx.y * warps + warp; head < heads_total; head += gridDim.y * warps)
    rope_one_head<T>(blockIdx.x, head, lane, qkv, q_out, positions, rope, qw, kw, has_norm, eps, H, Hkv, D,
                     k_cache, v_cache, slot_mapping, page_size, heads_total, ps);
}

// Two neighbouring pairs per lane and step, for the pairing (j, j + D/2) over the whole head
// with D / 2 even: 4- or 8-byte accesses, one cache line per warp and step.
template <typename T> struct Duo;
template <> struct Duo<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Duo<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

// What a (token, head) needs besides the head's values: where the result goes, the norm's weights
// and the angles of the token's position.  None of it is written by this step's kernels, so it is
// fetched before pdl_wait().
template <typename T, int STEPS>
struct RopeHead {
  T* dst;
  bool skip, is_v;
  float2 wa[STEPS], wb[STEPS], c[STEPS], sn[STEPS];
};

template <typename T, int STEPS>
__device__ __forceinline__ RopeHead<T, STEPS> rope_prepare_vec(int t, int head, int lane, T* __restrict__ q_out,
                                                               const int* __restrict__ positions, RopeArgs rope,
                                                               VecParam qw, VecParam kw, int has_norm, int H, int Hkv,
                                                               int D, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                               const int* __restrict__ slot_mapping, int page_size) {
  RopeHead<T, STEPS> h;
  h.skip = false;
  h.is_v = false;
  VecParam w = qw;
  if (head < H) {
    h.dst = q_out + ((size_t)t * H + head) * D;
  } else {
    const int slot = slot_mapping[t];
    h.skip = slot < 0;
    const int kvh = head < H + Hkv ? head - H : head - H - Hkv;
    h.is_v = head >= H + Hkv;
    const size_t page = h.skip ? 0 : slot / page_size, in_page = h.skip ? 0 : slot % page_size;
    h.dst = (h.is_v ? v_cache : k_cache) + ((page * Hkv + kvh) * page_size + in_page) * D;
    w = kw;
  }
  if (h.skip || h.is_v) return h;
  const int half = D >> 1;
  const int pos = positions[t];
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < half) {
      h.wa[s] = has_norm ? make_float2(w[j], w[j + 1]) : make_float2(1.f, 1.f);
      h.wb[s] = has_norm ? make_float2(w[half + j], w[half + j + 1]) : make_float2(1.f, 1.f);
      h.c[s] = *reinterpret_cast<const float2*>(rope.cos + (size_t)pos * half + j);
      h.sn[s] = *reinterpret_cast<const float2*>(rope.sin + (size_t)pos * half + j);
    }
  }
  return h;
}

template <typename T, int STEPS>
__device__ __forceinline__ void rope_apply_vec(const RopeHead<T, STEPS>& h, int t, int head, int lane,
                                               const T* __restrict__ qkv, int has_norm, float eps, int H, int Hkv,
                                               int D, PartialSrc ps) {
  if (h.skip) return;
  const T* src = qkv + (size_t)t * (H + 2 * Hkv) * D + (size_t)head * D;
  const int half = D >> 1;
  float2 a[STEPS], b[STEPS];
  float acc = 0.f;
  if (ps.base) {
    // the loads of all splits are issued before the first is used; the sum runs in split order
#pragma unroll
    for (int s = 0; s < STEPS; ++s) a[s] = b[s] = make_float2(0.f, 0.f);
    for (int k0 = 0; k0 < ps.splits; k0 += 4) {
      float2 qa[4][STEPS], qb[4][STEPS];
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (k0 + k < ps.splits && j < half) {
            qa[k][s] = __ldcg(reinterpret_cast<const float2*>(ps.base + ps.offset(k0 + k, t, head * D + j)));
            qb[k][s] = __ldcg(reinterpret_cast<const float2*>(ps.base + ps.offset(k0 + k, t, head * D + half + j)));
          }
        }
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (k0 + k < ps.splits && j < half) {
            a[s].x += qa[k][s].x; a[s].y += qa[k][s].y;
            b[s].x += qb[k][s].x; b[s].y += qb[k][s].y;
          }
        }
    }
  } else {
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int j = 2 * (lane + 32 * s);
      if (j < half) {
        a[s] = Duo<T>::load(src + j);
        b[s] = Duo<T>::load(src + half + j);
      }
    }
  }
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < half) acc += a[s].x * a[s].x + a[s].y * a[s].y + b[s].x * b[s].x + b[s].y * b[s].y;
  }
  if (h.is_v) {
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int j = 2 * (lane + 32 * s);
      if (j < half) {
        Duo<T>::store(h.dst + j, a[s].x, a[s].y);
        Duo<T>::store(h.dst + half + j, b[s].x, b[s].y);
      }
    }
    return;
  }
  const float rstd = has_norm ? rsqrtf(warp_sum(acc) / (float)D + eps) : 1.f;
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < half) {
      float a0 = a[s].x, a1 = a[s].y, b0 = b[s].x, b1 = b[s].y;
      if (has_norm) {
        a0 *= rstd * h.wa[s].x; a1 *= rstd * h.wa[s].y;
        b0 *= rstd * h.wb[s].x; b1 *= rstd * h.wb[s].y;
      }
      const float2 c = h.c[s], sn = h.sn[s];
      Duo<T>::store(h.dst + j, a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
      Duo<T>::store(h.dst + half + j, b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
    }
  }
}

template <typename T, int STEPS>
__global__ void qk_norm_rope_kvwrite_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                                const int* __restrict__ positions, RopeArgs rope,
                                                VecParam qw, VecParam kw, int has_norm, float eps,
                                                int H, int Hkv, int D, T* __restrict__ k_cache,
                                                T* __restrict__ v_cache,
                                                const int* __restrict__ slot_mapping, int page_size,
                                                int heads_total, PartialSrc ps) {
  pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, first = blockIdx.y * warps + warp;
  RopeHead<T, STEPS> h;
  if (first < heads_total)
    h = rope_prepare_vec<T, STEPS>(t, first, lane, q_out, positions, rope, qw, kw, has_norm, H, Hkv, D, k_cache,
                                   v_cache, slot_mapping, page_size);
  pdl_wait();
  for (int head = first; head < heads_total; head += gridDim.y * warps) {
    if (head != first)
      h = rope_prepare_vec<T, STEPS>(t, head, lane, q_out, positions, rope, qw, kw, has_norm, H, Hkv, D, k_cache,
                                     v_cache, slot_mapping, page_size);
    rope_apply_vec<T, STEPS>(h, t, head, lane, qkv, has_norm, eps, H, Hkv, D, ps);
  }
}

// Many tokens (prefill): a block per token whose warps walk the token's heads, ROPE_UNROLL heads
// at a time, so that each warp has that many heads' loads in flight; the token's angles and the
// norms' weights are fetched once per lane, not once per head.
constexpr int ROPE_UNROLL = 3;

template <typename T, int STEPS>
__global__ void qk_norm_rope_kvwrite_rows_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                                 const int* __restrict__ positions, RopeArgs rope,
                                                 VecParam qw, VecParam kw, int has_norm, float eps,
                                                 int H, int Hkv, int D, T* __restrict__ k_cache,
                                                 T* __restrict__ v_cache,
                                                 const int* __restrict__ slot_mapping, int page_size,
                                                 int heads_total) {
  pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, half = D >> 1;
  const int pos = positions[t];
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  float2 c[STEPS], sn[STEPS], wqa[STEPS], wqb[STEPS], wka[STEPS], wkb[STEPS];
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < half) {
      c[s] = *reinterpret_cast<const float2*>(rope.cos + (size_t)pos * half + j);
      sn[s] = *reinterpret_cast<const float2*>(rope.sin + (size_t)pos * half + j);
      wqa[s] = has_norm ? make_float2(qw[j], qw[j + 1]) : make_float2(1.f, 1.f);
      wqb[s] = has_norm ? make_float2(qw[half + j], qw[half + j + 1]) : make_float2(1.f, 1.f);
      wka[s] = has_norm ? make_float2(kw[j], kw[j + 1]) : make_float2(1.f, 1.f);
      wkb[s] = has_norm ? make_float2(kw[half + j], kw[half + j + 1]) : make_float2(1.f, 1.f);
    }
  }
  pdl_wait();
  const size_t page = slot >= 0 ? slot / page_size : 0, in_page = slot >= 0 ? slot % page_size : 0;
  const T* row = qkv + (size_t)t * (H + 2 * Hkv) * D;
  for (int h0 = warp; h0 < heads_total; h0 += warps * ROPE_UNROLL) {
    float2 a[ROPE_UNROLL][STEPS], b[ROPE_UNROLL][STEPS];
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int head = h0 + u * warps;
      if (head < heads_total) {
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (j < half) {
            a[u][s] = Duo<T>::load(row + (size_t)head * D + j);
            b[u][s] = Duo<T>::load(row + (size_t)head * D + half + j);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int head = h0 + u * warps;
      if (head >= heads_total) break;
      const bool is_q = head < H, is_v = head >= H + Hkv;
      if (!is_q && slot < 0) continue;
      const int kvh = is_q ? 0 : (is_v ? head - H - Hkv : head - H);
      T* dst = is_q ? q_out + ((size_t)t * H + head) * D
                    : (is_v ? v_cache : k_cache) + ((page * Hkv + kvh) * page_size + in_page) * D;
      if (is_v) {
#pragma unroll
        for (int s = 0; s < STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (j < half) {
            Duo<T>::store(dst + j, a[u][s].x, a[u][s].y);
            Duo<T>::store(dst + half + j, b[u][s].x, b[u][s].y);
          }
        }
        continue;
      }
      float acc = 0.f;
#pragma unroll
      for (int s = 0; s < STEPS; ++s) {
        const int j = 2 * (lane + 32 * s);
        if (j < half) acc += a[u][s].x * a[u][s].x + a[u][s].y * a[u][s].y + b[u][s].x * b[u][s].x + b[u][s].y * b[u][s].y;
      }
      const float rstd = has_norm ? rsqrtf(warp_sum(acc) / (float)D + eps) : 1.f;
#pragma unroll
      for (int s = 0; s < STEPS; ++s) {
        const int j = 2 * (lane + 32 * s);
        if (j < half) {
          const float2 wa = is_q ? wqa[s] : wka[s], wb = is_q ? wqb[s] : wkb[s];
          float a0 = a[u][s].x, a1 = a[u][s].y, b0 = b[u][s].x, b1 = b[u][s].y;
          if (has_norm) {
            a0 *= rstd * wa.x; a1 *= rstd * wa.y;
            b0 *= rstd * wb.x; b1 *= rstd * wb.y;
          }
          Duo<T>::store(dst + j, a0 * c[s].x - b0 * sn[s].x, a1 * c[s].y - b1 * sn[s].y);
          Duo<T>::store(dst + half + j, b0 * c[s].x + a0 * sn[s].x, b1 * c[s].y + a1 * sn[s].y);
        }
      }
    }
  }
}

// The same for head sizes 64, 128 and 256, with four neighbouring elements of each half per lane
// (8- or 16-byte accesses): LPH = D / 8 lanes share a head, a warp works on 32 / LPH heads at once.
template <typename T, int LPH>
__global__ void qk_norm_rope_kvwrite_rows4_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                                  const int* __restrict__ positions, RopeArgs rope,
                                                  VecParam qw, VecParam kw, int has_norm, float eps,
                                                  int H, int Hkv, T* __restrict__ k_cache,
                                                  T* __restrict__ v_cache,
                                                  const int* __restrict__ slot_mapping, int page_size,
                                                  int heads_total) {
  constexpr int D = LPH * 8, HALF = D / 2, HPW = 32 / LPH, U = 3;
  pdl_trigger();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, j = 4 * (lane % LPH);
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  float c[4], sn[4], wqa[4], wqb[4], wka[4], wkb[4];
  Quad<float>::load(rope.cos + (size_t)pos * HALF + j, c);
  Quad<float>::load(rope.sin + (size_t)pos * HALF + j, sn);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    wqa[e] = has_norm ? qw[j + e] : 1.f;
    wqb[e] = has_norm ? qw[HALF + j + e] : 1.f;
    wka[e] = has_norm ? kw[j + e] : 1.f;
    wkb[e] = has_norm ? kw[HALF + j + e] : 1.f;
  }
  pdl_wait();
  const size_t page = slot >= 0 ? slot / page_size : 0, in_page = slot >= 0 ? slot % page_size : 0;
  const T* row = qkv + (size_t)t * (H + 2 * Hkv) * D;
  for (int base = warp * HPW; base < heads_total; base += warps * HPW * U) {
    float a[U][4], b[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int head = base + sub + u * warps * HPW;
      if (head < heads_total) {
        Quad<T>::load(row + (size_t)head * D + j, a[u]);
        Quad<T>::load(row + (size_t)head * D + HALF + j, b[u]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) a[u][e] = b[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int head = base + sub + u * warps * HPW;
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc += a[u][e] * a[u][e] + b[u][e] * b[u][e];
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (head >= heads_total) continue;
      const bool is_q = head < H, is_v = head >= H + Hkv;
      if (!is_q && slot < 0) continue;
      const int kvh = is_q ? 0 : (is_v ? head - H - Hkv : head - H);
      T* dst = is_q ? q_out + ((size_t)t * H + head) * D
                    : (is_v ? v_cache : k_cache) + ((page * Hkv + kvh) * page_size + in_page) * D;
      float oa[4], ob[4];
      if (is_v) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { oa[e] = a[u][e]; ob[e] = b[u][e]; }
      } else {
        const float rstd = has_norm ? rsqrtf(acc / (float)D + eps) : 1.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x0 = a[u][e], x1 = b[u][e];
          if (has_norm) {
            x0 *= rstd * (is_q ? wqa[e] : wka[e]);
            x1 *= rstd * (is_q ? wqb[e] : wkb[e]);
          }
          oa[e] = x0 * c[e] - x1 * sn[e];
          ob[e] = x1 * c[e] + x0 * sn[e];
        }
      }
      Quad<T>::store(dst + j, oa);
      Quad<T>::store(dst + HALF + j, ob);
    }
  }
}

TS_EXPORT int ts_qk_norm_rope_kvwrite(int dtype, const void* qkv, void* q_out, const int* positions,
                                      const float* cos, const float* sin, int rotary_dim,
                                      int interleaved, const void* q_weight, const void* k_weight,
                                      int weight_is_f32, float eps, int num_tokens, int H, int Hkv,
                                      int D, void* k_cache, void* v_cache, const int* slot_mapping,
                                      int page_size, const float* partials, int splits, int n_tiles,
                                      int t_tiles, int tile_t, cudaStream_t stream) {
  TS_REQUIRE(partials == nullptr || (splits > 0 && n_tiles * 128 >= (H + 2 * Hkv) * D && tile_t > 0),
             "qk_norm_rope_kvwrite: partial tiles do not fit the row length");
  TS_REQUIRE(partials == nullptr || D % 2 == 0, "qk_norm_rope_kvwrite: partial tiles need an even head size");
  PartialSrc ps{partials, splits, n_tiles, t_tiles, tile_t};
  TS_REQUIRE(num_tokens > 0 && H > 0 && Hkv > 0 && D > 0, "qk_norm_rope_kvwrite: empty input");
  TS_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 2 == 0,
             "qk_norm_rope_kvwrite: rotary_dim %d does not fit head size %d", rotary_dim, D);
  TS_REQUIRE((q_weight == nullptr) == (k_weight == nullptr),
             "qk_norm_rope_kvwrite: q and k norm weights come together");
  TS_REQUIRE(slot_mapping == nullptr || (k_cache && v_cache && page_size > 0),
             "qk_norm_rope_kvwrite: cache write without a cache");
  const int heads_total = slot_mapping ? H + 2 * Hkv : H;
  // few tokens: a warp per head (most blocks); many tokens: 8 warps walk a token's heads
  const int warps = num_tokens >= 256 ? 8 : 4;
  dim3 grid(num_tokens, num_tokens >= 256 ? 1 : (heads_total + warps - 1) / warps);
  RopeArgs rope{cos, sin, rotary_dim, interleaved};
  VecParam qw{q_weight, weight_is_f32}, kw{k_weight, weight_is_f32};
  const int has_norm = q_weight != nullptr;
  // the pairing (j, j + D/2) over the whole head, D / 2 even and at most 256: two pairs per lane
  const bool vec = rotary_dim == D && !interleaved && (D / 2) % 2 == 0 && D <= 512 &&
                   (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                    reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) % 8 == 0;
#define TS_ROPE_VEC(T, STEPS)                                                                          \
  TS_LAUNCH("qk_norm_rope_kvwrite", (qk_norm_rope_kvwrite_vec_kernel<T, STEPS>), grid, warps * 32, 0, stream, \
            (const T*)qkv, (T*)q_out, positions, rope, qw, kw, has_norm, eps, H, Hkv, D, (T*)k_cache,  \
            (T*)v_cache, slot_mapping, page_size, heads_total, ps)
#define TS_ROPE_ROWS(T, STEPS)                                                                         \
  TS_LAUNCH("qk_norm_rope_kvwrite", (qk_norm_rope_kvwrite_rows_kernel<T, STEPS>), dim3(num_tokens), warps * 32, 0, \
            stream, (const T*)qkv, (T*)q_out, positions, rope, qw, kw, has_norm, eps, H, Hkv, D, (T*)k_cache, \
            (T*)v_cache, slot_mapping, page_size, heads_total)
#define TS_ROPE_ROWS4(T, LPH)                                                                         \
  TS_LAUNCH("qk_norm_rope_kvwrite", (qk_norm_rope_kvwrite_rows4_kernel<T, LPH>), dim3(num_tokens), warps * 32, 0, \
            stream, (const T*)qkv, (T*)q_out, positions, rope, qw, kw, has_norm, eps, H, Hkv, (T*)k_cache,  \
            (T*)v_cache, slot_mapping, page_size, heads_total)
  const bool aligned16 = (reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                          reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                          reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin)) % 16 == 0;
  if (vec && aligned16 && num_tokens >= 256 && partials == nullptr && (D == 64 || D == 128 || D == 256) &&
      (dtype == TS_F32 || dtype == TS_BF16)) {
    if (dtype == TS_F32) {
      if (D == 64) TS_ROPE_ROWS4(float, 8); else if (D == 128) TS_ROPE_ROWS4(float, 16); else TS_ROPE_ROWS4(float, 32);
    } else {
      if (D == 64) TS_ROPE_ROWS4(__nv_bfloat16, 8); else if (D == 128) TS_ROPE_ROWS4(__nv_bfloat16, 16); else TS_ROPE_ROWS4(__nv_bfloat16, 32);
    }
    return 0;
  }
#undef TS_ROPE_ROWS4
  if (vec && num_tokens >= 256 && partials == nullptr && D <= 256 && (dtype == TS_F32 || dtype == TS_BF16)) {
    const int steps = (D / 4 + 31) / 32;
    if (dtype == TS_F32) {
      if (steps <= 1) TS_ROPE_ROWS(float, 1); else TS_ROPE_ROWS(float, 2);
    } else {
      if (steps <= 1) TS_ROPE_ROWS(__nv_bfloat16, 1); else TS_ROPE_ROWS(__nv_bfloat16, 2);
    }
    return 0;
  }
#undef TS_ROPE_ROWS
  if (vec && (dtype == TS_F32 || dtype == TS_BF16)) {
    const int steps = (D / 4 + 31) / 32;        // pairs of pairs per lane
    if (dtype == TS_F32) {
      if (steps <= 1) TS_ROPE_VEC(float, 1); else if (steps <= 2) TS_ROPE_VEC(float, 2); else TS_ROPE_VEC(float, 4);
    } else {
      if (steps <= 1) TS_ROPE_VEC(__nv_bfloat16, 1); else if (steps <= 2) TS_ROPE_VEC(__nv_bfloat16, 2); else TS_ROPE_VEC(__nv_bfloat16, 4);
    }
    return 0;
  }
#undef TS_ROPE_VEC
  if (dtype == TS_F32)
    TS_LAUNCH("qk_norm_rope_kvwrite", qk_norm_rope_kvwrite_kernel<float>, grid, warps * 32, 0, stream,
              (const float*)qkv, (float*)q_out, positions, rope, qw, kw, has_norm, eps, H, Hkv, D,
              (float*)k_cache, (float*)v_cache, slot_mapping, page_size, heads_total, ps);
  else if (dtype == TS_BF16)
    TS_LAUNCH("qk_norm_rope_kvwrite", qk_norm_rope_kvwrite_kernel<__nv_bfloat16>, grid, warps * 32, 0, stream,
              (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, positions, rope, qw, kw, has_norm, eps, H,
              Hkv, D, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping, page_size, heads_total, ps);
  else
    return ts_fail("qk_norm_rope_kvwrite: unknown dtype %d", dtype);
  return 0;
}
