// Paged, variable-length, causal grouped-query attention for prefill on the 5th-generation tensor
// cores, bfloat16, head size 64 or 128 (-DTS_HEAD_DIM).
//
// A block of 192 threads handles 128 rows = (query, head of one KV group) pairs of one request and
// walks its visible keys in tiles of 128:
//   warp 0   loads: the query tile once (3-D TMA over [token, head, dim]), then per key tile the K
//            and V pages of the request's block table (2-D TMA boxes of one page x 64 columns,
//            128-byte swizzle) into a ring of two stages;
//   warp 1   issues tcgen05.mma: S = Q K^T into tensor memory, and, once the probabilities are in
//            shared memory, O += P V (V as an N-contiguous operand) into tensor memory;
//   warps 2-5 one thread per row: read the row of S from tensor memory, mask (key j is visible to
//            the query at position p iff j <= p and, with a window W > 0, j > p - W: serve.py:668-680),
//            online softmax in 32-bit with exp2 (tinykernels.py:386-413, 993), write P as bfloat16
//            into swizzled shared memory, rescale the row of O when its maximum moved; at the end
//            divide O by the row sum and store it.
// Row maxima and sums never leave their thread, so there are no shuffles.  Every mbarrier wait is
// bounded (tcgen05.cuh); a block that gives up raises ts_attention_tcgen05_error.
#include "tcgen05.cuh"

#ifndef TS_HEAD_DIM
#error "compile with -DTS_HEAD_DIM=64 or 128"
#endif

TS_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int D = TS_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 prefill kernel takes head sizes 64 and 128");
constexpr int BM = 128;                      // rows of a block
constexpr int BN = 128;                      // keys of a tile
constexpr int THREADS = 192;
constexpr int STAGES = 2;
constexpr int DCH = D / 64;                  // 64-column chunks of a head
constexpr int CHUNK_BYTES = 128 * 128;       // 128 rows of 128 bytes
constexpr int Q_BYTES = DCH * CHUNK_BYTES;
constexpr int KV_BYTES = DCH * CHUNK_BYTES;  // one of K or V of a tile
constexpr int P_BYTES = (BN / 64) * CHUNK_BYTES;
constexpr int TMEM_COLS = 256;               // S: columns 0..127, O: 128..128+D
constexpr size_t SMEM = 1024 + Q_BYTES + 2 * STAGES * KV_BYTES + P_BYTES + 256;

struct TcAttnParams {
  bf16* out;                // [T, H, D]
  const int* block_table;   // [B, max_blocks]
  const int* cu_q;          // [B + 1]
  const int* kv_lens;       // [B]
  const int* tile_req;      // optional work list: request and first query of every block
  const int* tile_q0;
  int H, Hkv, page_shift, page_size, max_blocks;
  int heads_per_tile, queries_per_tile, head_tiles;
  int window;
  float scale_log2;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* Qs = smem;
  char* Ks = Qs + Q_BYTES;                       // [STAGES][KV_BYTES]
  char* Vs = Ks + STAGES * KV_BYTES;             // [STAGES][KV_BYTES]
  char* Ps = Vs + STAGES * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + P_BYTES);
  uint64_t* q_full = bars;                       // 1
  uint64_t* kv_full = bars + 1;                  // [STAGES]
  uint64_t* kv_empty = kv_full + STAGES;         // [STAGES]
  uint64_t* s_full = kv_empty + STAGES;          // S holds the scores of a tile
  uint64_t* s_free = s_full + 1;                 // the softmax threads have read S
  uint64_t* p_full = s_free + 1;                 // P is in shared memory, O is rescaled
  uint64_t* o_ready = p_full + 1;                // O holds the sum over the tiles so far
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_trigger();
  pdl_wait();
  // with a work list block x handles tile x; else blocks (tile, request) cover max_q_len and exit
  // where a request has fewer queries
  const int b = p.tile_req ? p.tile_req[blockIdx.x] : blockIdx.z;
  const int kvh = blockIdx.y / p.head_tiles, head_tile = blockIdx.y % p.head_tiles;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = p.tile_req ? p.tile_q0[blockIdx.x]
                            : (gridDim.x - 1 - blockIdx.x) * p.queries_per_tile;     // heavy blocks first
  if (q0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int G = p.H / p.Hkv, GT = p.heads_per_tile, QPT = p.queries_per_tile;
  const int g0 = head_tile * GT;
  const int nq = min(QPT, q_len - q0);
  const int n_valid = QPT > 1 ? nq * GT : min(GT, G - g0);
  const int pos0 = kv_len - q_len + q0;
  const int j_hi = min(kv_len, pos0 + nq);
  const int j_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_tile = j_lo / BN, end_tile = (j_hi + BN - 1) / BN;
  const int n_tiles = end_tile - first_tile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_free), 4);
    mbar_init(smem_u32(p_full), 4);
    mbar_init(smem_u32(o_ready), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + BN;

  if (warp == 0) {
    if (lane == 0) {
      // queries: rows (query, head) with the head fastest; one box per 64 columns
      const uint32_t qbar = smem_u32(q_full);
      mbar_expect_tx(qbar, DCH * 64 * 2 * GT * QPT);
      for (int c = 0; c < DCH; ++c)
        tma_load_3d(smem_u32(Qs + c * CHUNK_BYTES), &map_q, qbar, c * 64, kvh * G + g0, q_begin + q0);
      const int* bt = p.block_table + (size_t)b * p.max_blocks;
      const int pages_per_tile = BN >> p.page_shift;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % STAGES;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ((t / STAGES) & 1) ^ 1, abort_flag)) break;
        const uint32_t bar = smem_u32(&kv_full[s]);
        mbar_expect_tx(bar, 2 * KV_BYTES);
        const int j0 = (first_tile + t) * BN;
        for (int pg = 0; pg < pages_per_tile; ++pg) {
          const int j = j0 + (pg << p.page_shift);
          const int page = j < j_hi ? bt[j >> p.page_shift] : 0;          // past the end: the null page
          const int row = (page * p.Hkv + kvh) << p.page_shift;
          for (int c = 0; c < DCH; ++c) {
            const int off = s * KV_BYTES + c * CHUNK_BYTES + (pg << p.page_shift) * 128;
            tma_load_2d(smem_u32(Ks + off), &map_k, bar, c * 64, row);
            tma_load_2d(smem_u32(Vs + off), &map_v, bar, c * 64, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BM, BN, false);
      constexpr uint32_t idesc_pv = make_idesc(BM, D, true);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag);
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int s = t % STAGES;
        ok = mbar_wait(smem_u32(&kv_full[s]), (t / STAGES) & 1, abort_flag) &&
             mbar_wait(smem_u32(s_free), (t & 1) ^ 1, abort_flag);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t qa = smem_u32(Qs), ka = smem_u32(Ks + s * KV_BYTES), va = smem_u32(Vs + s * KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma(tmem_s, smem_desc(qa + (k / 4) * CHUNK_BYTES + (k % 4) * 32),
               smem_desc(ka + (k / 4) * CHUNK_BYTES + (k % 4) * 32), idesc_qk, k > 0 ? 1u : 0u);
        tcgen05_commit(smem_u32(s_full));
        ok = mbar_wait(smem_u32(p_full), t & 1, abort_flag);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t pa = smem_u32(Ps);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          umma(tmem_o, smem_desc(pa + (k / 4) * CHUNK_BYTES + (k % 4) * 32),
               smem_desc_mn(va + k * 16 * 128, CHUNK_BYTES), idesc_pv, (t > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(smem_u32(&kv_empty[s]));
        tcgen05_commit(smem_u32(o_ready));
      }
    }
  } else {
    // one thread per row
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const bool valid = r < n_valid;
    const int qi = QPT > 1 ? r / GT : 0, gg = QPT > 1 ? r % GT : r;
    const int pos = valid ? pos0 + qi : -1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int j0 = (first_tile + t) * BN;
      ok = mbar_wait(smem_u32(s_full), t & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const bool all_visible = j0 + BN - 1 <= pos && j0 >= lo;
      // the whole row of S into registers: four loads in flight, one wait
      float sv[BN];
#pragma unroll
      for (int c = 0; c < BN; c += 32) tmem_load32_nowait(tmem_s + lane_addr + c, sv + c);
      tmem_load_wait();
      // S is read: the next tile's scores may overwrite it
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_free));
      if (!all_visible) {
#pragma unroll
        for (int e = 0; e < BN; ++e) {
          const int j = j0 + e;
          if (!(j <= pos && j >= lo)) sv[e] = -INFINITY;
        }
      }
      // the row's maximum, four independent chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < BN; e += 4) {
        mx4[0] = fmaxf(mx4[0], sv[e]);
        mx4[1] = fmaxf(mx4[1], sv[e + 1]);
        mx4[2] = fmaxf(mx4[2], sv[e + 2]);
        mx4[3] = fmaxf(mx4[3], sv[e + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2(m - m_safe);
      // probabilities -> shared memory (bfloat16, rows of 128 bytes, 16-byte pieces exchanged by
      // the row's low three bits: the 128-byte swizzle of the MMA operand)
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BN; c += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float p0 = ex2(fmaf(sv[c + e], p.scale_log2, -m_safe));        // -inf gives 0
          const float p1 = ex2(fmaf(sv[c + e + 1], p.scale_log2, -m_safe));
          sum4[(e / 2) & 3] += p0 + p1;
          packed[e / 2] = pack2(p0, p1);
        }
        const int idx = ((c % 64) / 8) ^ (r & 7);
        *reinterpret_cast<uint4*>(Ps + (c / 64) * CHUNK_BYTES + r * 128 + idx * 16) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l = l * alpha + sum;
      m = m_new;
      if (t > 0) {
        // the sum so far must be complete before it is rescaled
        ok = mbar_wait(smem_u32(o_ready), (t - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        if (!__all_sync(0xffffffffu, alpha == 1.f)) {
          float ov[D];
#pragma unroll
          for (int c = 0; c < D; c += 32) tmem_load32_nowait(tmem_o + lane_addr + c, ov + c);
          tmem_load_wait();
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            float v[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = ov[c + e] * alpha;
            tmem_store32(tmem_o + lane_addr + c, v);
          }
          tmem_store_wait();
        }
      }
      fence_async_shared();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(p_full));
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(smem_u32(o_ready), (n_tiles - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_tiles > 0) {
      tcgen05_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + ((size_t)(q_begin + q0 + qi) * p.H + kvh * G + g0 + gg) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        float v[32];
        tmem_load32(tmem_o + lane_addr + c, v);
        if (valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>(dst + c + e) =
                make_uint4(pack2(v[e] * inv, v[e + 1] * inv), pack2(v[e + 2] * inv, v[e + 3] * inv),
                           pack2(v[e + 4] * inv, v[e + 5] * inv), pack2(v[e + 6] * inv, v[e + 7] * inv));
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_s), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

bool encode(CUtensorMap* map, void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
            const cuuint32_t* box) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, base, dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

TS_EXPORT int ts_attention_tcgen05_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// q, out [T, H, D]; caches [num_pages, Hkv, page_size, D]; bfloat16.  tile_req / tile_q0 (optional,
// num_tiles ints each): the request and the first query of every block of 128 / group queries.
TS_EXPORT int ts_paged_attention_tcgen05(const void* q, void* out, const void* k_cache, const void* v_cache,
                                         const int* block_table, const int* cu_q, const int* kv_lens,
                                         int num_tokens, int num_requests, int max_q_len, int H, int Hkv,
                                         int num_pages, int page_size, int max_blocks, float scale, int window,
                                         const int* tile_req, const int* tile_q0, int num_tiles,
                                         int tile_queries, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && num_requests > 0 && max_q_len > 0, "paged_attention_tcgen05: empty batch");
  TS_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0, "paged_attention_tcgen05: %d heads over %d KV heads", H, Hkv);
  TS_REQUIRE(page_size >= 8 && page_size <= BN && (page_size & (page_size - 1)) == 0,
             "paged_attention_tcgen05: page size %d must be a power of two from 8 to %d", page_size, BN);
  TS_REQUIRE(num_requests <= 65535, "paged_attention_tcgen05: more than 65535 requests");
  TS_REQUIRE(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 == 0,
             "paged_attention_tcgen05: operands must be 16-byte aligned");
  const int G = H / Hkv;
  TcAttnParams p;
  p.out = (bf16*)out; p.block_table = block_table; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.tile_req = tile_req; p.tile_q0 = tile_q0;
  p.H = H; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.window = window;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.heads_per_tile = G < BM ? G : BM;
  p.queries_per_tile = G < BM ? BM / G : 1;
  p.head_tiles = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  const long long gy = (long long)Hkv * p.head_tiles;
  TS_REQUIRE(gy <= 65535, "paged_attention_tcgen05: too many head tiles");

  CUtensorMap mq, mk, mv;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)p.heads_per_tile, (cuuint32_t)p.queries_per_tile};
    TS_REQUIRE(encode(&mq, const_cast<void*>(q), 3, dims, strides, box), "paged_attention_tcgen05: tensor map of q failed");
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * Hkv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    TS_REQUIRE(encode(&mk, const_cast<void*>(k_cache), 2, dims, strides, box), "paged_attention_tcgen05: tensor map of the keys failed");
    TS_REQUIRE(encode(&mv, const_cast<void*>(v_cache), 2, dims, strides, box), "paged_attention_tcgen05: tensor map of the values failed");
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return ts_fail("paged_attention_tcgen05: %s", cudaGetErrorString(e));
    configured = true;
  }
  TS_REQUIRE((tile_req == nullptr) == (tile_q0 == nullptr) && (tile_req == nullptr || num_tiles > 0),
             "paged_attention_tcgen05: the work list is incomplete");
  TS_REQUIRE(tile_req == nullptr || tile_queries == p.queries_per_tile,
             "paged_attention_tcgen05: the work list was cut for %d queries a block, the kernel takes %d",
             tile_queries, p.queries_per_tile);
  dim3 grid((max_q_len + p.queries_per_tile - 1) / p.queries_per_tile, (unsigned)gy, num_requests);
  if (tile_req) grid = dim3(num_tiles, (unsigned)gy, 1);
  TS_LAUNCH("attn_prefill_tcgen05", attn_prefill_tc_kernel, grid, THREADS, SMEM, stream, mq, mk, mv, p);
  return 0;
}
