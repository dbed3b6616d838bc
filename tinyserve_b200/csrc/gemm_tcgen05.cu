// out[M, N] = x[M, K] * W[N, K]^T for few tokens (M up to 128), bfloat16, on the 5th-generation
// tensor cores: the weight-streaming matrix product of decode steps.
//
// Roles are swapped against the usual tiling: a block takes 128 rows of W as the M side of
// tcgen05.mma (so the weights, which are nearly all the bytes, stream through the 128 lanes of
// the tensor core) and the tokens, padded to TILE_T in {16, 32, 64, 128}, as its N side.  The
// accumulator D[128 weight rows x TILE_T tokens] lives in tensor memory.  Per 64-wide slice of K
// one thread issues two TMA loads (W tile 128 x 64, x tile TILE_T x 64, 128-byte swizzle) into a
// ring of shared-memory stages guarded by mbarriers; four threads of four warps issue one
// tcgen05.mma (K = 16) each per slice, into an accumulator of their own, and commit the stage back
// to the loader.  (One thread can issue a tcgen05.mma every 196 cycles, however small the MMA:
// measured on B200.  Four issuing warps give four times the rate, which a block needs to keep
// up with its share of the memory bandwidth when few blocks stream a product.)
//
// Shapes with few row tiles (N = 4096: 32 tiles for 148 SMs) are also cut along K.  Every block
// then stores its partial tile to scratch and bumps the tile's counter; the block that arrives
// last adds the partials in split order (so the sum is the same every run) and writes the
// output.  Nobody waits for anybody.  Counters return to zero for the next call.
//
// Every mbarrier wait is bounded: if a wait runs out, the block raises the library's error flag
// (ts_gemm_tcgen05_error), lets its copies land, frees its tensor memory and returns.
// tinyserve leaves these products to cuBLAS (serve.py:847, 883, 916, 919, 1263).
#include "tcgen05.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

#ifndef TS_GEMM_RING_KB
#define TS_GEMM_RING_KB 110          // shared memory of a block's ring of stages
#endif

using bf16 = __nv_bfloat16;
constexpr int TILE_N = 128;          // weight rows of a block (MMA M)
constexpr int BK = 64;               // K elements of a stage: 128 bytes, one swizzle row
constexpr int ISSUERS = BK / 16;     // issuing threads: one per K step of a stage, each with its own accumulator
constexpr int THREADS = 32 * (1 + ISSUERS);      // warp 0 loads, warps 1..4 issue, warps 0..3 do the epilogue
constexpr int W_STAGE_BYTES = TILE_N * BK * 2;

struct GemmParams {
  void* out;            // [M, ldc] bfloat16 or float
  float* partials;      // split-K scratch: [splits][row tiles][token tiles][TILE_T][128]
  int* counters;        // [row tiles * token tiles], zero between calls
  int M, N, K, ldc;
  int splits, out_f32;
  // Rows of x that still lack their RMSNorm factor: x holds v * norm_weight, and the sums of v^2
  // lie in x_sumsq [x_tiles][SUMSQ_STRIDE] (one partial sum per 128 columns of v).  The factor
  // rsqrt(sum / K + x_eps) of a token scales its column of the result.
  const float* x_sumsq;
  int x_tiles;
  float x_eps;
  // The residual form (the K cuts of a row tile are one cluster): residual [M, N] += result;
  // hprime [M, N] = bfloat16(residual * norm_w); sumsq_out [row tile][SUMSQ_STRIDE] = sums of
  // residual^2 over the tile's 128 columns, for the product that reads hprime.
  float* residual;
  VecParam norm_w;
  bf16* hprime;
  float* sumsq_out;
  // Gated form (no K cuts, up to 64 tokens): the weight rows alternate in blocks of 64, gate rows
  // then the matching up rows, so a 128-row tile holds both; out [M, N / 2] = act(gate) * up.
  int gated_act;        // 0: off; else the activation's code + 1
  VecParam bias;        // [N] added to every token's result (plain output only); ptr null: none
};
constexpr int SUMSQ_STRIDE = 16;     // tokens of the residual form (one token tile of 16)

// instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = tile_t
__host__ __device__ constexpr uint32_t instr_desc(int tile_t) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(tile_t >> 3) << 17) |
         (static_cast<uint32_t>(TILE_N >> 4) << 24);
}
// The four K steps of a stage go to four accumulators, one per issuing thread, which the
// epilogue adds up.
template <int TILE_T> struct Accs { static constexpr int N = ISSUERS; };

template <int TILE_T>
__device__ __forceinline__ void tmem_load8_sum(uint32_t addr, float (&v)[8]) {
  tmem_load8(addr, v);
#pragma unroll
  for (int a = 1; a < Accs<TILE_T>::N; ++a) {
    float t[8];
    tmem_load8(addr + a * TILE_T, t);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] += t[i];
  }
}

template <int TILE_T> struct Cfg {
  static constexpr int X_STAGE_BYTES = TILE_T * BK * 2;
  static constexpr int STAGE_BYTES = W_STAGE_BYTES + X_STAGE_BYTES;
  // two blocks share an SM: the ring and the barriers of a block stay below 113 KB
  static constexpr int RING = TS_GEMM_RING_KB * 1024;
  static constexpr int STAGES = RING / STAGE_BYTES < 2 ? 2 : (RING / STAGE_BYTES > 8 ? 8 : RING / STAGE_BYTES);
  static constexpr int TMEM_COLS = Accs<TILE_T>::N * TILE_T < 32 ? 32 : Accs<TILE_T>::N * TILE_T;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

template <int TILE_T>
__global__ void __launch_bounds__(THREADS)
gemm_wx_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
  using C = Cfg<TILE_T>;
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* ctrl = smem + (size_t)C::STAGES * C::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctrl);            // [STAGES]
  uint64_t* empty = full + C::STAGES;                            // [STAGES]
  uint64_t* accum = empty + C::STAGES;                           // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* is_last = const_cast<int*>(abort_flag) + 1;

  __shared__ float row_scale[TILE_T];
  __shared__ float sum_scratch[33];

  pdl_trigger();
  const int n_tile = blockIdx.x, t_tile = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_total = (p.K + BK - 1) / BK;
  const int per = (kb_total + p.splits - 1) / p.splits;
  const int kb0 = split * per;
  const int nkb = max(0, min(kb_total, kb0 + per) - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), ISSUERS);       // every issuing thread commits its own MMA
    }
    mbar_init(smem_u32(accum), ISSUERS);
    *abort_flag = 0;
    *is_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (threadIdx.x == 0) {
    // loader: one slice of K per stage.  The weight tiles of the first round do not depend on
    // the predecessor kernel: they are fetched before pdl_wait(), the token tiles after it.
    const int pre = min(nkb, C::STAGES);
    for (int i = 0; i < pre; ++i) {
      const uint32_t bar = smem_u32(&full[i]);
      mbar_expect_tx(bar, C::STAGE_BYTES);
      tma_load_2d(smem_u32(smem + (size_t)i * C::STAGE_BYTES), &map_w, bar, (kb0 + i) * BK, n_tile * TILE_N);
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i)
      tma_load_2d(smem_u32(smem + (size_t)i * C::STAGE_BYTES + W_STAGE_BYTES), &map_x, smem_u32(&full[i]),
                  (kb0 + i) * BK, t_tile * TILE_T);
    int armed = pre;
    for (int i = pre; i < nkb; ++i) {
      const int s = i % C::STAGES;
      const uint32_t round = i / C::STAGES;
      if (!mbar_wait(smem_u32(&empty[s]), (round & 1) ^ 1, abort_flag)) break;
      const uint32_t bar = smem_u32(&full[s]);
      mbar_expect_tx(bar, C::STAGE_BYTES);
      char* stage = smem + (size_t)s * C::STAGE_BYTES;
      tma_load_2d(smem_u32(stage), &map_w, bar, (kb0 + i) * BK, n_tile * TILE_N);
      tma_load_2d(smem_u32(stage + W_STAGE_BYTES), &map_x, bar, (kb0 + i) * BK, t_tile * TILE_T);
      armed = i + 1;
    }
    timeline_mark(2);      // all loads issued
    if (*abort_flag) {
      // let the copies that are still in flight land before the block goes away
      for (int i = max(0, armed - C::STAGES); i < armed; ++i) {
        const uint32_t bar = smem_u32(&full[i % C::STAGES]);
        for (uint32_t w = 0; w < WAIT_LIMIT && !mbar_try_wait(bar, (i / C::STAGES) & 1); ++w) {}
      }
    }
  } else if (warp >= 1 && lane == 0) {
    // issuer `k` of four: the k-th K step (16 wide) of every stage, into accumulator k
    const int k = warp - 1;
    pdl_wait();
    const uint32_t idesc = instr_desc(TILE_T);
    const uint64_t desc0 = smem_desc(smem_u32(smem));
    const uint32_t acc = tmem_base + k * TILE_T;
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % C::STAGES;
      ok = mbar_spin_wait(smem_u32(&full[s]), (i / C::STAGES) & 1, abort_flag);
      if (!ok) break;
      tcgen05_fence_after();
      // one descriptor per operand and stage; a K step of 16 is 32 bytes = 2 address units on
      const uint64_t ad = desc0 + (uint64_t)s * (C::STAGE_BYTES >> 4), bd = ad + (W_STAGE_BYTES >> 4);
      umma(acc, ad + 2 * k, bd + 2 * k, idesc, i > 0 ? 1u : 0u);
      tcgen05_commit(smem_u32(&empty[s]));
    }
    if (ok && nkb > 0) tcgen05_commit(smem_u32(accum));
  } else {
    pdl_wait();
    // (lanes 1.. of warps 1..4: they do not issue, they have time for the rows' norm factors)
    const int idle = (warp - 1) * 31 + lane - 1;          // 0 .. 123 over the non-issuing lanes of warps 1..4
    if (p.x_sumsq != nullptr && warp >= 1) {
      for (int j = idle; j < TILE_T; j += 31 * ISSUERS) {
        const int m = t_tile * TILE_T + j;
        float sum = 0.f;
        if (m < p.M)
          for (int t = 0; t < p.x_tiles; ++t) sum += __ldcg(p.x_sumsq + (size_t)t * SUMSQ_STRIDE + m);
        row_scale[j] = rsqrtf(sum / (float)p.K + p.x_eps);
      }
    }
  }
  __syncthreads();
  const bool scaled = p.x_sumsq != nullptr;

  // epilogue: lane = weight row, columns = tokens
  bool have = nkb > 0;
  if (have) have = mbar_spin_wait(smem_u32(accum), 0, abort_flag);
  have = __all_sync(0xffffffffu, have);      // tcgen05.ld is warp-wide: decide per warp
  tcgen05_fence_after();
  // warps 0..3 own the 128 lanes of tensor memory (a warp reaches the quarter of its index mod 4);
  // warp 4 only takes part in the barriers
  const bool epi = warp < 4;
  have = have && epi;
  const int n = n_tile * TILE_N + warp * 32 + lane;
  const int t0 = t_tile * TILE_T;
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  if (p.residual != nullptr) {
    // residual form.  Every block of the cluster leaves its partial tile in its shared memory
    // (the ring is idle: all MMAs have completed); rank r then owns the tokens r, r + splits, ...:
    // it adds the ranks' partial sums in rank order, adds the residual, and writes the new
    // residual, its product with the norm's weight and the tile's sum of squares.
    float* red = reinterpret_cast<float*>(smem);               // [TILE_T][TILE_N]
#pragma unroll 1
    for (int c = 0; c < TILE_T; c += 8) {
      float v[8];
      if (have) tmem_load8_sum<TILE_T>(taddr + c, v);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      if (epi) {
#pragma unroll
        for (int i = 0; i < 8; ++i) red[(c + i) * TILE_N + threadIdx.x] = scaled ? v[i] * row_scale[c + i] : v[i];
      }
    }
    const float wn = (epi && n < p.N) ? p.norm_w[n] : 0.f;
    cluster_arrive();
    cluster_wait();
    for (int j = split; j < TILE_T && t0 + j < p.M; j += p.splits) {
      const int m = t0 + j;
      float part[8];
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (epi && s < p.splits) part[s] = cluster_load_f32(red + j * TILE_N + threadIdx.x, s);
      float sq = 0.f;
      if (epi && n < p.N) {
        float sum = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s < p.splits) sum += part[s];
        const float v = p.residual[(size_t)m * p.N + n] + sum;
        p.residual[(size_t)m * p.N + n] = v;
        p.hprime[(size_t)m * p.N + n] = __float2bfloat16_rn(v * wn);
        sq = v * v;
      }
      const float total = block_sum(sq, sum_scratch);
      if (threadIdx.x == 0) p.sumsq_out[(size_t)n_tile * SUMSQ_STRIDE + m] = total;
    }
    // no block leaves while a peer may still read its shared memory
    cluster_arrive();
    cluster_wait();
  } else if (p.gated_act != 0) {
    if constexpr (TILE_T <= 64) {
      // lanes 0..63 hold gate rows, lanes 64..127 the up rows of the same output columns: the up
      // half goes through shared memory (the ring is idle), the gate half activates and stores
      float acc[TILE_T];
#pragma unroll
      for (int c = 0; c < TILE_T; c += 8) {
        float v[8];
        if (have) tmem_load8_sum<TILE_T>(taddr + c, v);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c + i] = scaled ? v[i] * row_scale[c + i] : v[i];
      }
      float* up = reinterpret_cast<float*>(smem);               // [64][TILE_T + 1]
      if (warp >= 2 && epi) {
#pragma unroll
        for (int i = 0; i < TILE_T; ++i) up[(threadIdx.x - 64) * (TILE_T + 1) + i] = acc[i];
      }
      __syncthreads();
      const int col = n_tile * 64 + threadIdx.x, half_n = p.N / 2;
      if (warp < 2 && col < half_n) {
#pragma unroll
        for (int i = 0; i < TILE_T; ++i) {
          const int m = t0 + i;
          if (m < p.M)
            static_cast<bf16*>(p.out)[(size_t)m * p.ldc + col] =
                __float2bfloat16_rn(activate(acc[i], p.gated_act - 1) * up[threadIdx.x * (TILE_T + 1) + i]);
        }
      }
    }
  } else if (p.splits == 1) {
    const float bn = (p.bias.ptr != nullptr && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll 1
    for (int c = 0; c < TILE_T; c += 8) {
      float v[8];
      if (have) tmem_load8_sum<TILE_T>(taddr + c, v);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      if (scaled) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= row_scale[c + i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += bn;
      if (epi && n < p.N) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = t0 + c + i;
          if (m < p.M) {
            if (p.out_f32) static_cast<float*>(p.out)[(size_t)m * p.ldc + n] = v[i];
            else static_cast<bf16*>(p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v[i]);
          }
        }
      }
    }
  } else {
    const int tiles = gridDim.x * gridDim.y, tile = t_tile * gridDim.x + n_tile;
    float* mine = p.partials + ((size_t)split * tiles + tile) * (TILE_T * TILE_N);
#pragma unroll 1
    for (int c = 0; c < TILE_T; c += 8) {
      float v[8];
      if (have) tmem_load8_sum<TILE_T>(taddr + c, v);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      if (epi) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mine[(c + i) * TILE_N + warp * 32 + lane] = scaled ? v[i] * row_scale[c + i] : v[i];
      }
    }
    if (p.out != nullptr) {
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int before = atomicAdd(&p.counters[tile], 1);
        *is_last = before == p.splits - 1;
        if (*is_last) p.counters[tile] = 0;
      }
      __syncthreads();
      if (*is_last && epi) {
        __threadfence();
        const float* base = p.partials + (size_t)tile * (TILE_T * TILE_N);
        const size_t split_stride = (size_t)tiles * (TILE_T * TILE_N);
        const float bn = (p.bias.ptr != nullptr && n < p.N) ? p.bias[n] : 0.f;
        // eight columns at a time, so that eight chains of loads are in flight per thread
#pragma unroll 1
        for (int c0 = 0; c0 < TILE_T && t0 + c0 < p.M; c0 += 8) {
          float sum[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) sum[i] = bn;
          for (int s = 0; s < p.splits; ++s) {
            const float* src = base + s * split_stride + c0 * TILE_N + warp * 32 + lane;
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] += __ldcg(src + i * TILE_N);
          }
          if (n < p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int m = t0 + c0 + i;
              if (m < p.M) {
                if (p.out_f32) static_cast<float*>(p.out)[(size_t)m * p.ldc + n] = sum[i];
                else static_cast<bf16*>(p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(sum[i]);
              }
            }
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  timeline_mark(3);        // results stored
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------- host side
// rows x K bfloat16 matrix with leading dimension ld; boxes of box_rows x 64 elements
bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TILE_T>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wx_kernel<TILE_T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)Cfg<TILE_T>::SMEM);
    if (e != cudaSuccess) return ts_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
    configured = true;
  }
  if (p.residual != nullptr) {
    // the K cuts of a row tile are the blocks of one cluster
    cudaError_t e = ts_launch_cluster(gemm_wx_kernel<TILE_T>, grid, dim3(THREADS), Cfg<TILE_T>::SMEM, stream,
                                      dim3(1, 1, p.splits), mw, mx, p);
    if (e != cudaSuccess) return ts_fail("gemm_tcgen05 (clusters of %d): %s", p.splits, cudaGetErrorString(e));
    return 0;
  }
  TS_LAUNCH("gemm_tcgen05", gemm_wx_kernel<TILE_T>, grid, THREADS, Cfg<TILE_T>::SMEM, stream, mw, mx, p);
  return 0;
}

}  // namespace

// 1 if a block ever gave up on a wait since the library was loaded (reads device memory: syncs)
TS_EXPORT int ts_gemm_tcgen05_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// scratch floats that `splits` > 1 needs
TS_EXPORT long long ts_gemm_tcgen05_scratch(int M, int N, int splits) {
  const int tile_t = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  const long long tiles = (long long)((N + TILE_N - 1) / TILE_N) * ((M + tile_t - 1) / tile_t);
  return splits > 1 ? (long long)splits * tiles * tile_t * TILE_N : 0;
}

// x [M, K] (leading dimension ldx), w [N, K] (ldw), out [M, N] (ldc) bfloat16 or float.
// counters: at least (N / 128 rounded up) * (M tiles) ints, all zero, when splits > 1.
// out == nullptr (with splits > 1): only the partial tiles are produced, laid out
// [split][token tile][row tile][token in tile][row in tile]; a consumer kernel adds them up.
namespace {
int gemm_tiled(const void* x, const void* w, void* out, int M, int N, int K, long long ldx, long long ldw,
               long long ldc, int out_f32, int splits, float* partials, int* counters, const float* x_sumsq,
               int x_tiles, float x_eps, float* residual, const void* norm_w, int norm_w_is_f32, void* hprime,
               float* sumsq_out, int gated_act, const void* bias, int bias_is_f32, cudaStream_t stream);
}

// bias: [N] float or bfloat16 (bias_is_f32), added to every token's result; needs an output
// (not with out == nullptr, where only partial tiles are produced).  nullptr: none.
TS_EXPORT int ts_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                              long long ldw, long long ldc, int out_f32, int splits, float* partials,
                              int* counters, const void* bias, int bias_is_f32, cudaStream_t stream) {
  TS_REQUIRE(bias == nullptr || out != nullptr, "gemm_tcgen05: a bias needs an output, not partial tiles only");
  return gemm_tiled(x, w, out, M, N, K, ldx, ldw, ldc, out_f32, splits, partials, counters, nullptr, 0, 0.f,
                    nullptr, nullptr, 0, nullptr, nullptr, 0, bias, bias_is_f32, stream);
}

// The same product with extras.  The first two are for up to 16 tokens.
// x_sumsq != nullptr: x holds rows v * norm_weight that still lack their RMSNorm factor, and
// x_sumsq [x_tiles][16] the sums of v^2 over each 128 columns; every token's result is scaled by
// rsqrt(sum / K + x_eps).
// residual != nullptr (out, partials and counters unused; splits <= 8, the cuts of a row tile
// are one thread-block cluster): residual [M, N] (float, contiguous) += x w^T; hprime [M, N]
// (bfloat16) = residual * norm_w; sumsq_out [N / 128 rounded up][16] = the sums of residual^2
// over each 128 columns, for the product that takes hprime as its x.
// gated_act != 0 (up to 64 tokens, splits == 1, bfloat16 out [M, N / 2], ldc its leading
// dimension, N a multiple of 128): the rows of w alternate in blocks of 64, gate rows then the
// matching up rows; out = act(gate) * up with act = gated_act - 1 (0 SiLU, 1 GELU-tanh).
TS_EXPORT int ts_gemm_tcgen05_fused(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                    long long ldw, long long ldc, int out_f32, int splits, float* partials,
                                    int* counters, const float* x_sumsq, int x_tiles, float x_eps,
                                    float* residual, const void* norm_w, int norm_w_is_f32, void* hprime,
                                    float* sumsq_out, int gated_act, cudaStream_t stream) {
  TS_REQUIRE((x_sumsq == nullptr && residual == nullptr) || M <= SUMSQ_STRIDE,
             "gemm_tcgen05: the scaled-rows and residual forms take up to %d tokens, got %d", SUMSQ_STRIDE, M);
  TS_REQUIRE(gated_act == 0 || (gated_act <= 2 && M <= 64 && splits == 1 && out && !out_f32 && !residual && N % 128 == 0),
             "gemm_tcgen05: the gated form takes up to 64 tokens, no K cuts, a bfloat16 output and whole 128-row tiles");
  TS_REQUIRE(x_sumsq == nullptr || x_tiles > 0, "gemm_tcgen05: sums of squares without their tile count");
  TS_REQUIRE(residual == nullptr || (norm_w && hprime && sumsq_out && splits <= 8),
             "gemm_tcgen05: the residual form needs the norm's weight, both outputs and at most 8 cuts");
  return gemm_tiled(x, w, out, M, N, K, ldx, ldw, ldc, out_f32, splits, partials, counters, x_sumsq, x_tiles,
                    x_eps, residual, norm_w, norm_w_is_f32, hprime, sumsq_out, gated_act, nullptr, 0, stream);
}

namespace {
int gemm_tiled(const void* x, const void* w, void* out, int M, int N, int K, long long ldx, long long ldw,
               long long ldc, int out_f32, int splits, float* partials, int* counters, const float* x_sumsq,
               int x_tiles, float x_eps, float* residual, const void* norm_w, int norm_w_is_f32, void* hprime,
               float* sumsq_out, int gated_act, const void* bias, int bias_is_f32, cudaStream_t stream) {
  TS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: empty operand");
  TS_REQUIRE(M <= 65535 * 128, "gemm_tcgen05: too many rows");
  TS_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05: K and the leading dimensions must be multiples of 8 (16-byte rows for TMA), got K=%d", K);
  TS_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
  TS_REQUIRE(splits >= 1 && splits <= 64, "gemm_tcgen05: splits out of range");
  TS_REQUIRE(residual != nullptr || splits == 1 || (partials && (counters || out == nullptr)), "gemm_tcgen05: split-K needs scratch and counters");
  TS_REQUIRE(residual != nullptr || out != nullptr || splits > 1, "gemm_tcgen05: without an output the partial tiles must be asked for (splits > 1)");
  const int tile_t = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap mw, mx;
  TS_REQUIRE(make_map(&mw, w, N, K, ldw, TILE_N), "gemm_tcgen05: cuTensorMapEncodeTiled failed for the weights");
  TS_REQUIRE(make_map(&mx, x, M, K, ldx, tile_t), "gemm_tcgen05: cuTensorMapEncodeTiled failed for the activations");
  GemmParams p;
  p.out = out; p.partials = partials; p.counters = counters;
  p.M = M; p.N = N; p.K = K; p.ldc = (int)ldc; p.splits = splits; p.out_f32 = out_f32;
  p.x_sumsq = x_sumsq; p.x_tiles = x_tiles; p.x_eps = x_eps;
  p.residual = residual; p.norm_w = VecParam{norm_w, norm_w_is_f32};
  p.hprime = static_cast<bf16*>(hprime); p.sumsq_out = sumsq_out;
  p.gated_act = gated_act;
  p.bias = VecParam{bias, bias_is_f32};
  dim3 grid((N + TILE_N - 1) / TILE_N, (M + tile_t - 1) / tile_t, splits);
  switch (tile_t) {
    case 16: return launch<16>(mw, mx, p, grid, stream);
    case 32: return launch<32>(mw, mx, p, grid, stream);
    case 64: return launch<64>(mw, mx, p, grid, stream);
    default: return launch<128>(mw, mx, p, grid, stream);
  }
}
}  // namespace
