// Sampling from 32-bit logits, one block per row, everything on the device.
//
//   temperature == 0           -> argmax (serve.py:1521-1522)
//   temperature > 0            -> x = logit / temperature, optional top-k (keep the k largest),
//                                 optional top-p (keep a token iff the probability mass of the
//                                 tokens ranked before it is <= top_p), then Gumbel-max over the
//                                 kept tokens: argmax(x + g) (serve.py:1544-1547, 1575-1588;
//                                 tinykernels.py:1813-1859)
//   repetition penalty         -> ts_apply_repetition_penalty, before sampling (serve.py:1488-1497)
//
// The noise is counter-based, so a row's sample does not depend on the rest of the batch:
// token v of a row uses word v % 4 of Philox-4x32-10 with key (seed_lo, seed_hi) and counter
// (v / 4, step, stream_lo, stream_hi); u = ((word >> 9) + 0.5) * 2^-23; g = -log(-log(u)).
// tinyserve draws from torch's global generator instead (serve.py:1546, tinykernels.py:1866).
// Ties go to the lowest token id.  Top-k keeps every token that ties with the k-th largest.
#include "common.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__device__ __forceinline__ float gumbel(uint32_t word) {
  const float u = ((float)(word >> 9) + 0.5f) * 1.1920928955078125e-07f;   // 2^-23
  return -logf(-logf(u));
}

// order-preserving map from float to unsigned
__device__ __forceinline__ uint32_t sort_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best {
  float value;
  int index;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}
__device__ Best block_best(Best v, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, v.value, o);
    other.index = __shfl_xor_sync(0xffffffffu, v.index, o);
    v = better(v, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    Best t = lane < (blockDim.x >> 5) ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other;
      other.value = __shfl_xor_sync(0xffffffffu, t.value, o);
      other.index = __shfl_xor_sync(0xffffffffu, t.index, o);
      t = better(t, other);
    }
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

__device__ float block_max_f(float v, float* scratch) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

struct SampleArgs {
  const float* logits;      // [rows, row_stride]
  long long row_stride;
  int vocab;
  const float* temperature; // [rows]
  const int* top_k;         // [rows] or null; <= 0 means off
  const float* top_p;       // [rows] or null; >= 1 means off
  const unsigned long long* stream;   // [rows] request key of the noise
  const unsigned int* step;           // [rows] position counter of the noise
  unsigned long long seed;
  int* out;                 // [rows]
  int* slot_tokens;         // optional: the token also goes to slot_tokens[slots[row]]
  const int* slots;
};

__global__ void __launch_bounds__(THREADS) sample_kernel(SampleArgs a) {
  __shared__ Best best_scratch[32];
  __shared__ float f_scratch[33];
  __shared__ unsigned long long hist[256];
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_above;
  __shared__ unsigned long long sh_total;

  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float* x = a.logits + (size_t)row * a.row_stride;
  const int V = a.vocab;
  const float temp = a.temperature[row];

  if (!(temp > 0.f)) {   // greedy
    Best b{-INFINITY, 0x7fffffff};
    for (int v = threadIdx.x; v < V; v += THREADS) b = better(b, Best{x[v], v});
    b = block_best(b, best_scratch);
    if (threadIdx.x == 0) {
      a.out[row] = b.index;
      if (a.slot_tokens) a.slot_tokens[a.slots[row]] = b.index;
    }
    return;
  }
  const float inv_temp = 1.f / temp;
  const int k = a.top_k ? a.top_k[row] : 0;
  const float top_p = a.top_p ? a.top_p[row] : 1.f;
  uint32_t keep_from = 0;   // tokens with sort_key(x / temp) >= keep_from are kept

  if (k > 0 && k < V) {
    // radix select of the k-th largest key, one byte per pass
    uint32_t prefix = 0, mask = 0;
    unsigned long long remaining = (unsigned long long)k;
    for (int byte = 3; byte >= 0; --byte) {
      for (int i = threadIdx.x; i < 256; i += THREADS) hist[i] = 0ull;
      __syncthreads();
      for (int v = threadIdx.x; v < V; v += THREADS) {
        const uint32_t key = sort_key(x[v] * inv_temp);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * byte)) & 255u], 1ull);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned long long cum = 0;
        int chosen = 0;
        for (int b = 255; b >= 0; --b) {
          if (cum + hist[b] >= remaining) { chosen = b; break; }
          cum += hist[b];
        }
        sh_prefix = prefix | ((uint32_t)chosen << (8 * byte));
        sh_above = remaining - cum;
      }
      __syncthreads();
      prefix = sh_prefix;
      remaining = sh_above;
      mask |= 0xFFu << (8 * byte);
    }
    keep_from = prefix;
  }

  if (top_p < 1.f) {
    // weights exp(x - max) as 32.32 fixed point: sums are exact and order-independent
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < V; v += THREADS) {
      const float y = x[v] * inv_temp;
      if (sort_key(y) >= keep_from) mx = fmaxf(mx, y);
    }
    mx = block_max_f(mx, f_scratch);
    uint32_t prefix = 0, mask = 0;
    unsigned long long above = 0;
    for (int byte = 3; byte >= 0; --byte) {
      for (int i = threadIdx.x; i < 256; i += THREADS) hist[i] = 0ull;
      __syncthreads();
      for (int v = threadIdx.x; v < V; v += THREADS) {
        const float y = x[v] * inv_temp;
        const uint32_t key = sort_key(y);
        if (key >= keep_from && (key & mask) == prefix) {
          const unsigned long long w = (unsigned long long)(expf(y - mx) * 4294967296.f);
          atomicAdd(&hist[(key >> (8 * byte)) & 255u], w);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        if (byte == 3) {
          unsigned long long total = 0;
          for (int b = 0; b < 256; ++b) total += hist[b];
          sh_total = (unsigned long long)((double)top_p * (double)total);
        }
        const unsigned long long lim = sh_total;
        unsigned long long cum = above;
        int chosen = 0;
        for (int b = 255; b >= 0; --b) {
          if (cum + hist[b] > lim) { chosen = b; break; }
          cum += hist[b];
        }
        sh_prefix = prefix | ((uint32_t)chosen << (8 * byte));
        sh_above = cum;
      }
      __syncthreads();
      prefix = sh_prefix;
      above = sh_above;
      mask |= 0xFFu << (8 * byte);
    }
    keep_from = max(keep_from, prefix);
  }

  // Gumbel-max over the kept tokens
  const uint32_t k0 = (uint32_t)a.seed, k1 = (uint32_t)(a.seed >> 32);
  const unsigned long long stream = a.stream[row];
  const uint32_t step = a.step[row];
  Best b{-INFINITY, 0x7fffffff};
  for (int base = threadIdx.x * 4; base < V; base += THREADS * 4) {
    uint32_t c[4] = {(uint32_t)(base >> 2), step, (uint32_t)stream, (uint32_t)(stream >> 32)};
    philox4x32_10(c, k0, k1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = base + j;
      if (v < V) {
        const float y = x[v] * inv_temp;
        if (sort_key(y) >= keep_from) b = better(b, Best{y + gumbel(c[j]), v});
      }
    }
  }
  b = block_best(b, best_scratch);
  if (threadIdx.x == 0) {
    a.out[row] = b.index;
    if (a.slot_tokens) a.slot_tokens[a.slots[row]] = b.index;
  }
}

// logits[row, id] = logit > 0 ? logit / penalty : logit * penalty for every listed id (>= 0);
// the host lists each distinct recent token once.
__global__ void repetition_penalty_kernel(float* logits, long long row_stride, int vocab,
                                          const int* rows, const int* ids, int ids_per_row,
                                          const float* penalty) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  float* x = logits + (size_t)rows[r] * row_stride;
  const float p = penalty[r];
  for (int i = threadIdx.x; i < ids_per_row; i += blockDim.x) {
    const int id = ids[(size_t)r * ids_per_row + i];
    if (id >= 0 && id < vocab) {
      const float v = x[id];
      x[id] = v > 0.f ? v / p : v * p;
    }
  }
}

}  // namespace

TS_EXPORT int ts_sample(const float* logits, long long row_stride, int num_rows, int vocab,
                        const float* temperature, const int* top_k, const float* top_p,
                        const unsigned long long* stream_ids, const unsigned int* steps,
                        unsigned long long seed, int* out, int* slot_tokens, const int* slots,
                        cudaStream_t stream) {
  TS_REQUIRE(num_rows > 0 && vocab > 0, "sample: empty input");
  TS_REQUIRE(row_stride >= vocab, "sample: row stride smaller than the vocabulary");
  TS_REQUIRE(temperature && stream_ids && steps && out, "sample: missing argument");
  TS_REQUIRE((slot_tokens == nullptr) == (slots == nullptr), "sample: slot_tokens and slots come together");
  SampleArgs a{logits, row_stride, vocab, temperature, top_k, top_p, stream_ids, steps, seed, out, slot_tokens, slots};
  TS_LAUNCH("sample", sample_kernel, num_rows, THREADS, 0, stream, a);
  return 0;
}

TS_EXPORT int ts_apply_repetition_penalty(float* logits, long long row_stride, int vocab,
                                          const int* rows, const int* ids, int num_rows,
                                          int ids_per_row, const float* penalty,
                                          cudaStream_t stream) {
  TS_REQUIRE(num_rows > 0 && ids_per_row > 0, "repetition_penalty: empty input");
  TS_LAUNCH("repetition_penalty", repetition_penalty_kernel, num_rows, 256, 0, stream, logits, row_stride, vocab,
            rows, ids, ids_per_row, penalty);
  return 0;
}
