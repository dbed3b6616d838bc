// Paged grouped-query attention on the tensor cores for bfloat16, one head size per build
// (-DTS_HEAD_DIM=..., a multiple of 16 up to 256).
//
// Two kernels share the tile code:
//   prefill: a block of 4 warps handles 64 rows = (query, head of one KV group) pairs and walks
//            the visible keys in tiles of 64, K and V double-buffered in shared memory by cp.async;
//            tiles that lie wholly below a warp's rows skip the mask;
//   decode : requests that bring one token.  A block handles the heads of one KV group (up to 16
//            rows) and one of `num_splits` key ranges; its 4 warps take 16 keys each of every
//            64-key tile (3 stages in flight) and merge their partial softmax at the end.  Up
//            to 8 ranges are the blocks of a cluster and merge through distributed shared memory;
//            more are merged by attention_combine_kernel.
// Scores, running maxima, sums and the output accumulate in 32-bit; exp2 with scale * log2(e);
// the probabilities are rounded to bfloat16 for P * V, as tinykernels.py:386-413 and 993 do.
// Visibility as serve.py:668-680: key j is seen by the query at position p iff j <= p and, with a
// window W > 0, j > p - W.  Keys are found through the block table; the cache layout is
// [page, kv_head, slot, head_dim].
#include "tcgen05.cuh"

#ifndef TS_HEAD_DIM
#error "compile with -DTS_HEAD_DIM=<head size, a multiple of 16>"
#endif

TS_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int D = TS_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int CH = D / 8;                 // 16-byte chunks of a row
constexpr int ROW_BYTES = D * 2 + 16;     // rows are padded by one chunk: ldmatrix without conflicts
constexpr int THREADS = 128;              // decode block
#ifndef TS_PREFILL_WARPS
#define TS_PREFILL_WARPS 4
#endif
constexpr int PRE_THREADS = 32 * TS_PREFILL_WARPS;   // prefill block: warps of 16 rows each
constexpr int BN = 64;                    // keys of a tile
constexpr int BM = 16 * TS_PREFILL_WARPS; // rows of a prefill block
constexpr float LOG2E = 1.4426950408889634f;
constexpr bool Q_IN_REGS = D <= 128;

struct MmaAttnParams {
  const bf16* q;            // [T, H, D]
  bf16* out;                // [T, H, D]
  const bf16* k_cache;      // [pages, Hkv, page_size, D]
  const bf16* v_cache;
  const int* block_table;   // [B, max_blocks]
  const int* cu_q;          // [B + 1]
  const int* kv_lens;       // [B]
  const int* tile_req;      // optional work list: request and first query of every block
  const int* tile_q0;
  float* part_o;            // [T, H, splits, D]
  float* part_ml;           // [T, H, splits, 2]  (max in the log2 domain, sum)
  int cluster_merge;        // the key ranges of a (request, KV group) form a cluster and merge in shared memory
  int H, Hkv, page_shift, page_mask, max_blocks;
  int heads_per_tile, queries_per_tile, head_tiles;
  int num_splits, window;
  float scale_log2;
  // Decode straight from the fused q/k/v projection (from_qkv != 0; q is not read): every block
  // builds its query rows itself (sum of the split-K partial tiles, per-head RMSNorm, rotary), and
  // the block whose key range holds the newest position builds that key and value too, uses them
  // from shared memory and (head tile 0) writes them to the cache.
  int from_qkv;
  const bf16* qkv;          // [T, (H + 2 Hkv) * D], or null: the partial tiles in `ps`
  PartialSrc ps;
  const int* positions;     // [T]
  const int* slot_mapping;  // [T] cache slot of the token (page * page_size + row), -1: none
  const float* rope_cos;    // [positions, D / 2]
  const float* rope_sin;
  VecParam q_weight, k_weight;
  int has_norm;
  float eps;
  bf16* k_cache_out;        // the same caches, for the newest token's key and value
  bf16* v_cache_out;
};

// 16 bytes global -> shared; `valid` false writes zeros (the source is not read)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special function unit; -inf gives 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// NKEYS keys from j0 on -> shared memory (keys and values); keys outside [j_lo, j_hi) become zeros
template <int NKEYS, int NTHREADS>
__device__ __forceinline__ void load_kv_tile(char* ks, char* vs, const MmaAttnParams& p, const int* bt,
                                             int kvh, int j0, int j_lo, int j_hi) {
  for (int i = threadIdx.x; i < NKEYS * CH; i += NTHREADS) {
    const int key = i / CH, c = i % CH;
    const int j = j0 + key;
    const bool valid = j >= j_lo && j < j_hi;
    size_t off = 0;
    if (valid) {
      const size_t page = bt[j >> p.page_shift];
      off = (((page * p.Hkv + kvh) << p.page_shift) + (j & p.page_mask)) * D + c * 8;
    }
    cp_async16(smem_u32(ks + key * ROW_BYTES + c * 16), p.k_cache + off, valid);
    cp_async16(smem_u32(vs + key * ROW_BYTES + c * 16), p.v_cache + off, valid);
  }
}

// Where 16 bytes of a key or value tile lie in shared memory: row `key`, 16-byte piece `piece` of
// the row.  Padded rows (cp.async path), or, for tiles brought by TMA, 64-column chunks of
// 128-byte rows with the 128-byte swizzle (a piece changes place with the row's low three bits);
// both keep ldmatrix free of bank conflicts.
template <bool SWZ>
__device__ __forceinline__ uint32_t kv_piece(const char* tile, int key, int piece) {
  if (SWZ) return smem_u32(tile + (piece >> 3) * (BN * 128) + key * 128 + (((piece & 7) ^ (key & 7)) << 4));
  return smem_u32(tile + key * ROW_BYTES + piece * 16);
}

// S[16 x (8 * NT)] += Q[16 x D] * K^T for the NT*8 keys that start at row `key0` of the K tile.
// `qs` points at this warp's 16 query rows in shared memory (used when the fragments are not held
// in registers); `qf` holds them otherwise.
template <int NT, bool SWZ = false>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const char* qs, const uint32_t (*qf)[4],
                                        const char* ks, int key0, int lane) {
  static_assert(NT % 2 == 0, "key tiles come in pairs");
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kstep = 0; kstep < D / 16; ++kstep) {
    uint32_t a[4];
    if (Q_IN_REGS) {
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = qf[kstep][e];
    } else {
      ldmatrix_x4(a, smem_u32(qs + ((mi & 1) * 8 + r) * ROW_BYTES + (kstep * 2 + (mi >> 1)) * 16));
    }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, kv_piece<SWZ>(ks, key0 + np * 16 + (mi >> 1) * 8 + r, kstep * 2 + (mi & 1)));
      mma_bf16(s[2 * np], a, b[0], b[1]);
      mma_bf16(s[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x (8 * NT)] * V for the keys that start at row `key0` of the V tile
template <int NT, bool SWZ = false>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&s)[NT][4], const char* vs,
                                        int key0, int lane) {
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, kv_piece<SWZ>(vs, key0 + kk * 16 + (mi & 1) * 8 + r, dp * 2 + (mi >> 1)));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online softmax of one tile for the two rows a lane holds (g and g + 8 of the warp's 16).
// s holds raw scores on entry and probabilities on exit.  `jbase` is the position of column 0.
// pos[h] is the position of row h's query, lo[h] the lowest visible key; a row with pos < 0 sees
// nothing.
// MASK false: every key of the tile is visible to both rows (no comparisons).
template <int NT, bool MASK = true>
__device__ __forceinline__ void softmax_tile(float (&s)[NT][4], float (&o)[D / 8][4], float (&m)[2],
                                             float (&l)[2], const int (&pos)[2], const int (&lo)[2],
                                             int jbase, float scale_log2, int lane) {
  const int t = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = jbase + nt * 8 + 2 * t + e;
        const bool visible = !MASK || (j <= pos[h] && j >= lo[h]);
        const float v = visible ? s[nt][2 * h + e] * scale_log2 : -INFINITY;
        s[nt][2 * h + e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = fast_exp2(m[h] - m_safe);      // m[h] = -inf gives 0
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pr = fast_exp2(s[nt][2 * h + e] - m_safe);
        s[nt][2 * h + e] = pr;
        sum += pr;
      }
    l[h] = l[h] * alpha + sum;       // the four lanes of a row are added up at the end
    m[h] = m_new;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][2 * h] *= alpha;
      o[dt][2 * h + 1] *= alpha;
    }
  }
}

// ------------------------------------------------------------------ prefill (any q_len)
__global__ void __launch_bounds__(PRE_THREADS) attn_prefill_kernel(MmaAttnParams p) {
  extern __shared__ __align__(16) char smem[];
  char* Qs = smem;                           // [BM][ROW_BYTES]
  char* Ks = Qs + BM * ROW_BYTES;            // [2][BN][ROW_BYTES]
  char* Vs = Ks + 2 * BN * ROW_BYTES;        // [2][BN][ROW_BYTES]

  pdl_trigger();
  pdl_wait();
  // with a work list block x handles tile x; else blocks (tile, request) cover max_q_len and exit
  // where a request has fewer queries (the last queries see the most keys: their blocks go first)
  const int b = p.tile_req ? p.tile_req[blockIdx.x] : blockIdx.z;
  const int kvh = blockIdx.y / p.head_tiles, head_tile = blockIdx.y % p.head_tiles;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = p.tile_req ? p.tile_q0[blockIdx.x] : (gridDim.x - 1 - blockIdx.x) * p.queries_per_tile;
  if (q0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int G = p.H / p.Hkv, GT = p.heads_per_tile, QPT = p.queries_per_tile;
  const int g0 = head_tile * GT;
  const int nq = min(QPT, q_len - q0);
  const int n_valid = QPT > 1 ? nq * GT : min(GT, G - g0);      // valid rows are a prefix
  const int pos0 = kv_len - q_len + q0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int* bt = p.block_table + (size_t)b * p.max_blocks;

  for (int i = threadIdx.x; i < BM * CH; i += PRE_THREADS) {
    const int r = i / CH, c = i % CH;
    const bool valid = r < n_valid;
    const int qi = QPT > 1 ? r / GT : 0, gg = QPT > 1 ? r % GT : r;
    const bf16* src = valid ? p.q + ((size_t)(q_begin + q0 + qi) * p.H + kvh * G + g0 + gg) * D + c * 8 : p.q;
    cp_async16(smem_u32(Qs + r * ROW_BYTES + c * 16), src, valid);
  }
  const int j_hi = min(kv_len, pos0 + nq);
  const int j_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_tile = j_lo / BN, end_tile = (j_hi + BN - 1) / BN;
  load_kv_tile<BN, PRE_THREADS>(Ks, Vs, p, bt, kvh, first_tile * BN, j_lo, j_hi);
  cp_async_commit();

  int pos[2], lo[2];
  int warp_max_pos = -1, warp_min_pos = -1, warp_max_lo = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    pos[h] = r < n_valid ? pos0 + (QPT > 1 ? r / GT : 0) : -1;
    lo[h] = p.window > 0 ? max(0, pos[h] - p.window + 1) : 0;
  }
  {
    const int last = min(warp * 16 + 15, n_valid - 1);
    if (last >= warp * 16) {
      warp_max_pos = pos0 + (QPT > 1 ? last / GT : 0);
      // a tile needs no mask if all 16 rows of the warp are valid and see all of its keys
      if (last == warp * 16 + 15) warp_min_pos = pos0 + (QPT > 1 ? (warp * 16) / GT : 0);
      warp_max_lo = p.window > 0 ? max(0, warp_max_pos - p.window + 1) : 0;
    }
  }
  float o[D / 8][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
  uint32_t qf[Q_IN_REGS ? D / 16 : 1][4];
  const char* my_q = Qs + warp * 16 * ROW_BYTES;

  for (int tile = first_tile; tile < end_tile; ++tile) {
    const int buf = (tile - first_tile) & 1;
    if (tile + 1 < end_tile)
      load_kv_tile<BN, PRE_THREADS>(Ks + (buf ^ 1) * BN * ROW_BYTES, Vs + (buf ^ 1) * BN * ROW_BYTES, p, bt,
                                    kvh, (tile + 1) * BN, j_lo, j_hi);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (Q_IN_REGS && tile == first_tile) {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int kstep = 0; kstep < D / 16; ++kstep)
        ldmatrix_x4(qf[kstep], smem_u32(my_q + ((mi & 1) * 8 + r) * ROW_BYTES + (kstep * 2 + (mi >> 1)) * 16));
    }
    if (tile * BN <= warp_max_pos) {      // a warp whose rows all stand before this tile skips it
      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      qk_tile<BN / 8>(s, my_q, qf, Ks + buf * BN * ROW_BYTES, 0, lane);
      if (tile * BN + BN - 1 <= warp_min_pos && tile * BN >= warp_max_lo)
        softmax_tile<BN / 8, false>(s, o, m, l, pos, lo, tile * BN, p.scale_log2, lane);
      else
        softmax_tile<BN / 8, true>(s, o, m, l, pos, lo, tile * BN, p.scale_log2, lane);
      pv_tile<BN / 8>(o, s, Vs + buf * BN * ROW_BYTES, 0, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (r >= n_valid) continue;
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    const int qi = QPT > 1 ? r / GT : 0, gg = QPT > 1 ? r % GT : r;
    bf16* dst = p.out + ((size_t)(q_begin + q0 + qi) * p.H + kvh * G + g0 + gg) * D;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
      *reinterpret_cast<__nv_bfloat162*>(dst + dt * 8 + 2 * t) =
          __floats2bfloat162_rn(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
  }
}

// ------------------------------------------------------------------ decode (q_len == 1)
constexpr int DEC_STAGES = 3;
constexpr int ROPE_STEPS = (D / 4 + 31) / 32;      // pairs of pairs per lane over half a head

// What a lane needs of the norm weights and of the rotary angles of a position, for its elements
// of a head (pairs j, j + 1 of both halves): fetched before the dependency wait.
struct HeadConsts {
  float2 wa[ROPE_STEPS], wb[ROPE_STEPS], c[ROPE_STEPS], sn[ROPE_STEPS];
};
__device__ __forceinline__ void load_weights(HeadConsts& h, const VecParam& w, bool has_norm, int lane) {
  constexpr int HALF = D / 2;
#pragma unroll
  for (int s = 0; s < ROPE_STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    h.wa[s] = h.wb[s] = make_float2(1.f, 1.f);
    if (has_norm && j < HALF) {
      h.wa[s] = make_float2(w[j], w[j + 1]);
      h.wb[s] = make_float2(w[HALF + j], w[HALF + j + 1]);
    }
  }
}
__device__ __forceinline__ void load_angles(HeadConsts& h, const MmaAttnParams& p, int pos, int lane) {
  constexpr int HALF = D / 2;
#pragma unroll
  for (int s = 0; s < ROPE_STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    h.c[s] = h.sn[s] = make_float2(0.f, 0.f);
    if (j < HALF) {
      h.c[s] = *reinterpret_cast<const float2*>(p.rope_cos + (size_t)pos * HALF + j);
      h.sn[s] = *reinterpret_cast<const float2*>(p.rope_sin + (size_t)pos * HALF + j);
    }
  }
}

// One head of token t of the fused projection (column `col0` on, D wide), by one warp: the sum of
// the partial tiles (or the plain row), RMSNorm over the head with the weights in `h` (has_norm),
// rotary with the pairing (j, j + D / 2) (rotate), rounded to bfloat16, to `dst` (shared memory).
// The arithmetic is that of qk_norm_rope_kvwrite (elementwise.cu), so both paths agree bit by bit.
__device__ __forceinline__ void build_head(const MmaAttnParams& p, int t, int col0, bool rotate, const HeadConsts& h,
                                           int lane, bf16* dst) {
  constexpr int HALF = D / 2;
  float2 a[ROPE_STEPS], b[ROPE_STEPS];
#pragma unroll
  for (int s = 0; s < ROPE_STEPS; ++s) a[s] = b[s] = make_float2(0.f, 0.f);
  if (p.ps.base) {
    // the loads of up to eight splits are in flight together; the sum runs in split order
    for (int k0 = 0; k0 < p.ps.splits; k0 += 8) {
      float2 qa[8][ROPE_STEPS], qb[8][ROPE_STEPS];
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int s = 0; s < ROPE_STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (k0 + k < p.ps.splits && j < HALF) {
            qa[k][s] = __ldcg(reinterpret_cast<const float2*>(p.ps.base + p.ps.offset(k0 + k, t, col0 + j)));
            qb[k][s] = __ldcg(reinterpret_cast<const float2*>(p.ps.base + p.ps.offset(k0 + k, t, col0 + HALF + j)));
          }
        }
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int s = 0; s < ROPE_STEPS; ++s) {
          const int j = 2 * (lane + 32 * s);
          if (k0 + k < p.ps.splits && j < HALF) {
            a[s].x += qa[k][s].x; a[s].y += qa[k][s].y;
            b[s].x += qb[k][s].x; b[s].y += qb[k][s].y;
          }
        }
    }
  } else {
    const bf16* src = p.qkv + (size_t)t * (p.H + 2 * p.Hkv) * D + col0;
#pragma unroll
    for (int s = 0; s < ROPE_STEPS; ++s) {
      const int j = 2 * (lane + 32 * s);
      if (j < HALF) {
        a[s] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + j));
        b[s] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + HALF + j));
      }
    }
  }
  if (!rotate) {       // a value head: copied as it is
#pragma unroll
    for (int s = 0; s < ROPE_STEPS; ++s) {
      const int j = 2 * (lane + 32 * s);
      if (j < HALF) {
        *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(a[s].x, a[s].y);
        *reinterpret_cast<__nv_bfloat162*>(dst + HALF + j) = __floats2bfloat162_rn(b[s].x, b[s].y);
      }
    }
    return;
  }
  float acc = 0.f;
#pragma unroll
  for (int s = 0; s < ROPE_STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < HALF) acc += a[s].x * a[s].x + a[s].y * a[s].y + b[s].x * b[s].x + b[s].y * b[s].y;
  }
  const float rstd = p.has_norm ? rsqrtf(warp_sum(acc) / (float)D + p.eps) : 1.f;
#pragma unroll
  for (int s = 0; s < ROPE_STEPS; ++s) {
    const int j = 2 * (lane + 32 * s);
    if (j < HALF) {
      float a0 = a[s].x, a1 = a[s].y, b0 = b[s].x, b1 = b[s].y;
      if (p.has_norm) {
        a0 *= rstd * h.wa[s].x; a1 *= rstd * h.wa[s].y;
        b0 *= rstd * h.wb[s].x; b1 *= rstd * h.wb[s].y;
      }
      const float2 c = h.c[s], sn = h.sn[s];
      *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
      *reinterpret_cast<__nv_bfloat162*>(dst + HALF + j) = __floats2bfloat162_rn(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
    }
  }
}

// TMA false: key and value tiles come by cp.async, 16 bytes a thread, into padded rows (any head
// size in steps of 16, any page size).  TMA true (head sizes in steps of 64, pages of 32 or 64
// keys): one thread fetches whole pages as boxes of page x 64 columns with the 128-byte swizzle
// and an mbarrier per stage counts their bytes; an SM streams about half as much again this way
// as through its load/store unit's miss queue.  Whole pages come, also the keys past the
// request's length in its last page: those are masked, and must hold finite numbers (the engine's
// cache starts as zeros and only ever takes keys and values).
template <bool TMA>
__device__ __forceinline__ void attn_decode_body(const MmaAttnParams& p, const CUtensorMap* map_k,
                                                 const CUtensorMap* map_v) {
  extern __shared__ __align__(16) char smem[];
  constexpr int KV_TILE = TMA ? BN * D * 2 : BN * ROW_BYTES;      // bytes of the keys (or values) of a stage
  char* Qs = smem;                                   // [16][ROW_BYTES]
  char* Ks = TMA ? reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(Qs + 16 * ROW_BYTES) + 1023) & ~uintptr_t(1023))
                 : Qs + 16 * ROW_BYTES;              // [DEC_STAGES][KV_TILE]
  char* Vs = Ks + DEC_STAGES * KV_TILE;              // [DEC_STAGES][KV_TILE]
  __shared__ uint64_t full[DEC_STAGES];              // (TMA) the stage's bytes have landed
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  if (TMA && threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(smem_u32(&full[s]), 1);
    abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (TMA) __syncthreads();

  pdl_trigger();
  // The lengths, the block table and every cached key but the newest were written before this
  // step's kernels began: the first tiles are fetched before pdl_wait(), while the kernels that
  // make this token's query, key and value still run.  The tile with the newest key and the
  // query follow after it.
  // with a request list block z handles its entry z (the one-token requests of a mixed batch)
  const int b = p.tile_req ? p.tile_req[blockIdx.z] : blockIdx.z, split = blockIdx.y;
  const int kvh = blockIdx.x / p.head_tiles, head_tile = blockIdx.x % p.head_tiles;
  const int q_begin = p.cu_q[b];
  if (p.cu_q[b + 1] - q_begin != 1) return;
  const int kv_len = p.kv_lens[b];
  const int G = p.H / p.Hkv, g0 = head_tile * 16, ng = min(16, G - g0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  const int* bt = p.block_table + (size_t)b * p.max_blocks;
  const int qpos = kv_len - 1;
  const int j_hi = kv_len, j_lo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
  const int first_tile = j_lo / BN, total = (j_hi + BN - 1) / BN - first_tile;
  const int per_split = (total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = first_tile + split * per_split;
  const int n_tiles = max(0, min(first_tile + total, tile_begin + per_split) - tile_begin);
  const int newest_tile = qpos / BN;
  // from the projection itself the newest key never comes from the cache: every tile may be
  // fetched before the wait, without that key, which this block makes itself
  const bool from_qkv = p.from_qkv != 0;
  const int j_load = from_qkv ? j_hi - 1 : j_hi;
  const int late_tile = from_qkv ? -1 : newest_tile;
  const bool has_newest = from_qkv && newest_tile >= tile_begin && newest_tile < tile_begin + n_tiles;
  __shared__ __align__(16) bf16 newest_kv[2 * D];

  // tile `tile` of the keys and values into stage `stage`
  auto load_tile = [&](int stage, int tile, int j_end) {
    if (TMA) {
      // the boxes of a tile (pages x 64-column chunks x keys/values) are dealt to the lanes of
      // warp 0, so that issuing them costs the block one box's time, not sixteen; lane 0's
      // arrival carries the tile's byte count, so the stage cannot complete before it
      if (threadIdx.x < 32) {
        const int pages_per_tile = BN >> p.page_shift, boxes = pages_per_tile * (D / 64) * 2;
        const uint32_t bar = smem_u32(&full[stage]);
        if (threadIdx.x == 0) mbar_expect_tx(bar, 2 * KV_TILE);
        __syncwarp();
        for (int i = threadIdx.x; i < boxes; i += 32) {
          const int values = i & 1, c = (i >> 1) % (D / 64), pg = (i >> 1) / (D / 64);
          const int j = tile * BN + (pg << p.page_shift);
          const int page = j < j_hi ? bt[j >> p.page_shift] : 0;                        // past the end: the null page
          const int row = (page * p.Hkv + kvh) << p.page_shift;
          const int off = stage * KV_TILE + c * (BN * 128) + (pg << p.page_shift) * 128;
          tma_load_2d(smem_u32((values ? Vs : Ks) + off), values ? map_v : map_k, bar, c * 64, row);
        }
      }
    } else {
      load_kv_tile<BN, THREADS>(Ks + stage * KV_TILE, Vs + stage * KV_TILE, p, bt, kvh, tile * BN, j_lo, j_end);
    }
  };
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s)
    if (s < n_tiles && tile_begin + s != late_tile) load_tile(s, tile_begin + s, j_load);
  // the timeline build follows the blocks of one (request, KV group): marks 40.. with the key
  // range as their value
  const bool traced = blockIdx.x == 0 && blockIdx.z == 0 && threadIdx.x == 0;
  if (traced) timeline_mark_thread(40, split);          // first tiles on their way
  int slot = -1;
  HeadConsts hq, hk;
  if (from_qkv) {
    const int pos_q = p.positions[q_begin];
    slot = p.slot_mapping[q_begin];
    load_angles(hq, p, pos_q, lane);
    load_weights(hq, p.q_weight, p.has_norm, lane);
    hk = hq;
    if (has_newest) load_weights(hk, p.k_weight, p.has_norm, lane);
  }
  if (traced) timeline_mark_thread(41, split);          // constants fetched
  pdl_wait();
  if (traced) timeline_mark_thread(42, split);          // the projection is there
  if (from_qkv) {
    // the heads this block makes, dealt to the warps in turn: the newest key (norm, rotary) and
    // value where this block holds them, then the query rows; rows past the group are zero
    const int extra = has_newest ? 2 : 0;
    for (int i = warp; i < extra + 16; i += THREADS / 32) {
      if (i < extra) {
        build_head(p, q_begin, (p.H + (i == 0 ? 0 : p.Hkv) + kvh) * D, i == 0, hk, lane, newest_kv + i * D);
        continue;
      }
      const int r = i - extra;
      bf16* row = reinterpret_cast<bf16*>(Qs + r * ROW_BYTES);
      if (r < ng) {
        build_head(p, q_begin, (kvh * G + g0 + r) * D, true, hq, lane, row);
      } else {
        for (int d = lane * 2; d < D; d += 64) *reinterpret_cast<uint32_t*>(row + d) = 0u;
      }
    }
    __syncthreads();
    if (has_newest && head_tile == 0 && slot >= 0) {
      const size_t page = slot >> p.page_shift, in_page = slot & p.page_mask;
      const size_t at = (((page * p.Hkv + kvh) << p.page_shift) + in_page) * D;
      for (int d = threadIdx.x * 2; d < 2 * D; d += THREADS * 2) {
        bf16* dst = d < D ? p.k_cache_out + at + d : p.v_cache_out + at + (d - D);
        *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(newest_kv + d);
      }
    }
  } else {
    for (int i = threadIdx.x; i < 16 * CH; i += THREADS) {
      const int r = i / CH, c = i % CH;
      const bool valid = r < ng;
      const bf16* src = valid ? p.q + ((size_t)q_begin * p.H + kvh * G + g0 + r) * D + c * 8 : p.q;
      cp_async16(smem_u32(Qs + r * ROW_BYTES + c * 16), src, valid);
    }
  }
#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < n_tiles && tile_begin + s == late_tile) load_tile(s, tile_begin + s, j_hi);
    // the first group holds the query and all of these tiles; the others stay empty, so that the
    // loop below finds as many groups as it counts on
    cp_async_commit();
  }
  if (TMA) {        // only the query rows came by cp.async
    cp_async_wait<0>();
    __syncthreads();
  }
  if (traced) timeline_mark_thread(43, split);          // query rows (and the newest key) made
  int pos[2], lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    pos[h] = g + 8 * h < ng ? qpos : -1;
    lo[h] = j_lo;
  }
  float o[D / 8][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
  uint32_t qf[Q_IN_REGS ? D / 16 : 1][4];

  for (int it = 0; it < n_tiles; ++it) {
    const int nxt = it + DEC_STAGES - 1;
    if (nxt < n_tiles) load_tile(nxt % DEC_STAGES, tile_begin + nxt, j_load);
    if (TMA) {
      // bounded; a wait that ran out raises the block's abort flag and the status word, the loop
      // goes on over whatever the stage holds, and the block stores no output at the end
      mbar_wait(smem_u32(&full[it % DEC_STAGES]), (it / DEC_STAGES) & 1, abort_flag);
    } else {
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();
    }
    __syncthreads();
    if (has_newest && tile_begin + it == newest_tile) {
      // the newest key and value take their row of the tile (the copy left zeros or stale bytes there)
      const int row = qpos - newest_tile * BN, buf_n = it % DEC_STAGES;
      for (int d = threadIdx.x * 2; d < 2 * D; d += THREADS * 2) {
        const int e = d < D ? d : d - D;          // element of the head; two neighbours per thread
        char* tile = (d < D ? Ks : Vs) + (size_t)buf_n * KV_TILE;
        char* dst = TMA ? tile + (e / 64) * (BN * 128) + row * 128 + ((((e % 64) / 8) ^ (row & 7)) << 4) + (e % 8) * 2
                        : tile + row * ROW_BYTES + e * 2;
        *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(newest_kv + d);
      }
      __syncthreads();
    }
    if (Q_IN_REGS && it == 0) {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int kstep = 0; kstep < D / 16; ++kstep)
        ldmatrix_x4(qf[kstep], smem_u32(Qs + ((mi & 1) * 8 + r) * ROW_BYTES + (kstep * 2 + (mi >> 1)) * 16));
    }
    const int buf = it % DEC_STAGES;
    const int jbase = (tile_begin + it) * BN + warp * 16;
    if (jbase < j_hi) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      qk_tile<2, TMA>(s, Qs, qf, Ks + buf * KV_TILE, warp * 16, lane);
      softmax_tile<2>(s, o, m, l, pos, lo, jbase, p.scale_log2, lane);
      pv_tile<2, TMA>(o, s, Vs + buf * KV_TILE, warp * 16, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  if (traced) timeline_mark_thread(44, split);          // all key tiles done

  // merge the four warps' partial softmax through shared memory (the K buffers are free now)
  float* sm_o = reinterpret_cast<float*>(Ks);                  // [4][16][D]
  float* sm_ml = sm_o + 4 * 16 * D;                            // [4][16][2]
  float* cl_ml = sm_ml + 4 * 16 * 2;                           // [16][2] of the block, for its cluster
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int r = g + 8 * h;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      sm_o[(warp * 16 + r) * D + dt * 8 + 2 * (lane & 3)] = o[dt][2 * h];
      sm_o[(warp * 16 + r) * D + dt * 8 + 2 * (lane & 3) + 1] = o[dt][2 * h + 1];
    }
    if ((lane & 3) == 0) {
      sm_ml[(warp * 16 + r) * 2] = m[h];
      sm_ml[(warp * 16 + r) * 2 + 1] = sum;
    }
  }
  __syncthreads();
  const bool stores = !TMA || abort_flag_s == 0;
  for (int i = threadIdx.x; i < ng * D; i += THREADS) {
    const int r = i / D, d = i % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, sm_ml[(w * 16 + r) * 2]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_ml[(w * 16 + r) * 2];
      const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - mx);
      num = fmaf(wgt, sm_o[(w * 16 + r) * D + d], num);
      den = fmaf(wgt, sm_ml[(w * 16 + r) * 2 + 1], den);
    }
    const int head = kvh * G + g0 + r;
    if (p.num_splits == 1) {
      if (stores) p.out[((size_t)q_begin * p.H + head) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else if (p.cluster_merge) {
      // this thread has read its four values of (r, d); the first warp's place now holds their sum
      sm_o[r * D + d] = num;
      if (d == 0) {
        cl_ml[r * 2] = mx;
        cl_ml[r * 2 + 1] = den;
      }
    } else {
      // partial rows go by token, or by the entry of the request list when there is one
      const size_t row = (size_t)(p.tile_req ? (int)blockIdx.z : q_begin) * p.H + head;
      p.part_o[(row * p.num_splits + split) * D + d] = num;
      if (d == 0) {
        p.part_ml[(row * p.num_splits + split) * 2] = mx;
        p.part_ml[(row * p.num_splits + split) * 2 + 1] = den;
      }
    }
  }
  if (p.cluster_merge) {
    // The blocks of a (request, KV group) are one cluster, rank = key range.  Each block merges
    // its share of the (head, dimension) pairs from all ranks' shared memory, in rank order.
    cluster_arrive();
    cluster_wait();
    const int per_rank = (ng * D + p.num_splits - 1) / p.num_splits;
    const int i_end = min(ng * D, (split + 1) * per_rank);
    for (int i = split * per_rank + threadIdx.x; i < i_end; i += THREADS) {
      const int r = i / D, d = i % D;
      float ms[8], ls[8], os[8];
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < p.num_splits) {
          ms[s] = cluster_load_f32(cl_ml + r * 2, s);
          ls[s] = cluster_load_f32(cl_ml + r * 2 + 1, s);
          os[s] = cluster_load_f32(sm_o + r * D + d, s);
        }
      float mx = -INFINITY;
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < p.num_splits) mx = fmaxf(mx, ms[s]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < p.num_splits) {
          const float wgt = ms[s] == -INFINITY ? 0.f : exp2f(ms[s] - mx);
          num = fmaf(wgt, os[s], num);
          den = fmaf(wgt, ls[s], den);
        }
      if (stores) p.out[((size_t)q_begin * p.H + kvh * G + g0 + r) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
    if (traced) timeline_mark_thread(45, split);        // merged and stored
    // no block leaves while a peer may still read its shared memory
    cluster_arrive();
    cluster_wait();
    if (traced) timeline_mark_thread(46, split);
    return;
  }
}

__global__ void __launch_bounds__(THREADS) attn_decode_kernel(MmaAttnParams p) {
  attn_decode_body<false>(p, nullptr, nullptr);
}
constexpr bool TMA_HEAD = D % 64 == 0;        // boxes are 64 columns wide
__global__ void __launch_bounds__(THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       MmaAttnParams p) {
  attn_decode_body<TMA_HEAD>(p, &map_k, &map_v);
}

// out[row] = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s over the key ranges of a row
// (block x merges partial row x into output row x, or into head x % H of token tokens[x / H];
// a negative token marks an unused entry of the list)
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, int num_splits, int H,
                                         const int* __restrict__ tokens) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  if (tokens && tokens[blockIdx.x / H] < 0) return;
  const size_t out_row = tokens ? (size_t)tokens[blockIdx.x / H] * H + blockIdx.x % H : row;
  const float* ml = part_ml + row * num_splits * 2;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, ml[2 * s]);
  float den = 0.f;
  for (int s = 0; s < num_splits; ++s) den += ml[2 * s] == -INFINITY ? 0.f : exp2f(ml[2 * s] - mx) * ml[2 * s + 1];
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = ml[2 * s] == -INFINITY ? 0.f : exp2f(ml[2 * s] - mx);
      v = fmaf(w, part_o[(row * num_splits + s) * D + d], v);
    }
    out[out_row * D + d] = __float2bfloat16_rn(v * inv);
  }
}

}  // namespace

TS_EXPORT int ts_attention_mma_head_dim() { return D; }

// 1 if a block of the TMA decode kernel ever gave up on a wait since the library was loaded
// (reads device memory: synchronises)
TS_EXPORT int ts_attention_mma_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// decode_only != 0: every request brings one token (requests with another count are skipped);
// decode_only == 2: up to 8 key ranges are merged through the distributed shared
// memory of a cluster (no scratch is touched, no second launch);
// num_splits > 1 needs scratch: part_o T*H*splits*D floats, part_ml T*H*splits*2 floats.
// tile_req / tile_q0 (optional, num_tiles ints each): for the prefill kernel the request and the
// first query of every block of tile_queries queries; with decode_only the one-token requests of
// a mixed batch and their tokens (the scratch then has num_tiles rows in place of T).
// Key ranges that are no cluster are merged by a second launch.
namespace {
int paged_attention_mma_impl(const MmaAttnParams* from_qkv, const void* q, void* out, const void* k_cache,
                             const void* v_cache, const int* block_table, const int* cu_q, const int* kv_lens,
                             int num_tokens, int num_requests, int max_q_len, int H, int Hkv, int page_size,
                             int max_blocks, float scale, int window, int num_splits, float* part_o,
                             float* part_ml, int decode_only, const int* tile_req,
                             const int* tile_q0, int num_tiles, int tile_queries, int num_pages, cudaStream_t stream);
}

TS_EXPORT int ts_paged_attention_mma(const void* q, void* out, const void* k_cache, const void* v_cache,
                                     const int* block_table, const int* cu_q, const int* kv_lens,
                                     int num_tokens, int num_requests, int max_q_len, int H, int Hkv,
                                     int page_size, int max_blocks, float scale, int window,
                                     int num_splits, float* part_o, float* part_ml,
                                     int decode_only, const int* tile_req, const int* tile_q0, int num_tiles,
                                     int tile_queries, int num_pages, cudaStream_t stream) {
  return paged_attention_mma_impl(nullptr, q, out, k_cache, v_cache, block_table, cu_q, kv_lens, num_tokens,
                                  num_requests, max_q_len, H, Hkv, page_size, max_blocks, scale, window, num_splits,
                                  part_o, part_ml, decode_only, tile_req, tile_q0, num_tiles,
                                  tile_queries, num_pages, stream);
}

// Decode (every request brings one token) straight from the fused q/k/v projection: qkv
// [T, (H + 2 Hkv) * D] bfloat16, or null with the projection's split-K partial tiles (partials,
// splits, n_tiles, t_tiles, tile_t as gemm_tcgen05.cu leaves them).  The kernel applies the
// per-head RMSNorm (q_weight, k_weight of D elements, bfloat16 or float; null: none) and the
// rotary encoding (cos, sin [positions, D / 2], pairing (j, j + D / 2) over the whole head) itself
// and writes the token's key and value to slot_mapping[t] of the caches.  merge: 1 a combine
// launch (scratch as for ts_paged_attention_mma), 2 clusters (up to 8 key ranges).
TS_EXPORT int ts_paged_attention_mma_from_qkv(const void* qkv, const float* partials, int splits, int n_tiles,
                                              int t_tiles, int tile_t, const int* positions,
                                              const int* slot_mapping, const float* cos, const float* sin,
                                              const void* q_weight, const void* k_weight, int weight_is_f32,
                                              float eps, void* out, void* k_cache, void* v_cache,
                                              const int* block_table, const int* cu_q, const int* kv_lens,
                                              int num_tokens, int num_requests, int H, int Hkv, int page_size,
                                              int max_blocks, float scale, int window, int num_splits,
                                              float* part_o, float* part_ml, int merge, int num_pages,
                                              cudaStream_t stream) {
  TS_REQUIRE((qkv != nullptr) != (partials != nullptr), "paged_attention_mma_from_qkv: the projection or its partial tiles");
  TS_REQUIRE(partials == nullptr || (splits > 0 && n_tiles * 128 >= (H + 2 * Hkv) * D && tile_t > 0),
             "paged_attention_mma_from_qkv: partial tiles do not fit the row length");
  TS_REQUIRE(positions && slot_mapping && cos && sin && k_cache && v_cache,
             "paged_attention_mma_from_qkv: positions, slots, rotary tables and caches are needed");
  TS_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "paged_attention_mma_from_qkv: q and k norm weights come together");
  TS_REQUIRE(merge == 1 || merge == 2, "paged_attention_mma_from_qkv: merge is 1 (launch) or 2 (cluster)");
  MmaAttnParams extra = {};
  extra.from_qkv = 1;
  extra.qkv = static_cast<const bf16*>(qkv);
  extra.ps = PartialSrc{partials, splits, n_tiles, t_tiles, tile_t};
  extra.positions = positions; extra.slot_mapping = slot_mapping;
  extra.rope_cos = cos; extra.rope_sin = sin;
  extra.q_weight = VecParam{q_weight, weight_is_f32}; extra.k_weight = VecParam{k_weight, weight_is_f32};
  extra.has_norm = q_weight != nullptr; extra.eps = eps;
  extra.k_cache_out = static_cast<bf16*>(k_cache); extra.v_cache_out = static_cast<bf16*>(v_cache);
  return paged_attention_mma_impl(&extra, nullptr, out, k_cache, v_cache, block_table, cu_q, kv_lens, num_tokens,
                                  num_requests, 1, H, Hkv, page_size, max_blocks, scale, window, num_splits, part_o,
                                  part_ml, merge, nullptr, nullptr, 0, 0, num_pages, stream);
}

namespace {
int paged_attention_mma_impl(const MmaAttnParams* from_qkv, const void* q, void* out, const void* k_cache,
                             const void* v_cache, const int* block_table, const int* cu_q, const int* kv_lens,
                             int num_tokens, int num_requests, int max_q_len, int H, int Hkv, int page_size,
                             int max_blocks, float scale, int window, int num_splits, float* part_o,
                             float* part_ml, int decode_only, const int* tile_req,
                             const int* tile_q0, int num_tiles, int tile_queries, int num_pages, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && num_requests > 0 && max_q_len > 0, "paged_attention_mma: empty batch");
  TS_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0, "paged_attention_mma: %d heads over %d KV heads", H, Hkv);
  TS_REQUIRE(page_size > 0 && (page_size & (page_size - 1)) == 0, "paged_attention_mma: page size %d is no power of two", page_size);
  TS_REQUIRE(num_splits >= 1 && num_splits <= 64, "paged_attention_mma: num_splits %d out of range", num_splits);
  TS_REQUIRE(num_splits == 1 || (decode_only && ((part_o && part_ml) || (decode_only == 2 && num_splits <= 8))),
             "paged_attention_mma: splits are for decode and need scratch");
  TS_REQUIRE(num_requests <= 65535, "paged_attention_mma: more than 65535 requests");
  MmaAttnParams p = from_qkv ? *from_qkv : MmaAttnParams{};
  p.q = (const bf16*)q; p.out = (bf16*)out; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_table = block_table; p.cu_q = cu_q; p.kv_lens = kv_lens; p.part_o = part_o; p.part_ml = part_ml;
  p.cluster_merge = 0;
  p.tile_req = tile_req;
  p.tile_q0 = tile_q0;
  TS_REQUIRE((tile_req == nullptr) == (tile_q0 == nullptr) && (tile_req == nullptr || num_tiles > 0),
             "paged_attention_mma: the work list is incomplete");
  p.H = H; p.Hkv = Hkv; p.max_blocks = max_blocks;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.page_mask = page_size - 1;
  p.num_splits = num_splits; p.window = window; p.scale_log2 = scale * LOG2E;
  const int G = H / Hkv;
  cudaError_t e;
  if (decode_only) {
    p.heads_per_tile = 16; p.queries_per_tile = 1; p.head_tiles = (G + 15) / 16;
    // whole pages by TMA where the sizes allow it
    // (pages of 32 and 64 keys: measured on B200, 64 requests x 4096 keys, pages of 64: 6.67 TB/s by
    // TMA against 5.78 by cp.async; with pages of 16 both reach 5.4: the 4 KB pieces are what limits)
    const bool tma = TMA_HEAD && num_pages > 0 && page_size >= 32 && page_size <= BN &&
                     ((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0;
    CUtensorMap mk, mv;
    if (tma) {
      EncodeTiledFn fn = encode_tiled();
      TS_REQUIRE(fn != nullptr, "paged_attention_mma: the driver's tensor-map encoder was not found");
      const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * Hkv * page_size};
      const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
      const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
      const cuuint32_t elem[2] = {1, 1};
      for (int i = 0; i < 2; ++i)
        TS_REQUIRE(fn(i ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(i ? v_cache : k_cache), dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "paged_attention_mma: cuTensorMapEncodeTiled failed for the cache");
    }
    const size_t smem = tma ? (size_t)16 * ROW_BYTES + 1024 + (size_t)2 * DEC_STAGES * BN * D * 2
                            : (size_t)(16 + 2 * DEC_STAGES * BN) * ROW_BYTES;
    static bool configured = false, configured_tma = false;
    if (!(tma ? configured_tma : configured)) {
      e = tma ? cudaFuncSetAttribute(attn_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
              : cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return ts_fail("paged_attention_mma: %s", cudaGetErrorString(e));
      (tma ? configured_tma : configured) = true;
    }
    // tile_req / tile_q0 here: the one-token requests of a mixed batch and their tokens
    const int count = tile_req ? num_tiles : num_requests;
    dim3 grid(Hkv * p.head_tiles, num_splits, count);
    if (decode_only == 2 && num_splits > 1 && num_splits <= 8) {
      p.cluster_merge = 1;
      e = tma ? ts_launch_cluster(attn_decode_tma_kernel, grid, dim3(THREADS), smem, stream, dim3(1, num_splits, 1), mk, mv, p)
              : ts_launch_cluster(attn_decode_kernel, grid, dim3(THREADS), smem, stream, dim3(1, num_splits, 1), p);
      if (e != cudaSuccess) return ts_fail("attn_decode (clusters of %d): %s", num_splits, cudaGetErrorString(e));
      return 0;
    }
    if (tma) TS_LAUNCH("attn_decode_tma", attn_decode_tma_kernel, grid, THREADS, smem, stream, mk, mv, p);
    else TS_LAUNCH("attn_decode", attn_decode_kernel, grid, THREADS, smem, stream, p);
    if (num_splits > 1) {
      TS_LAUNCH("attention_combine", attention_combine_kernel, (tile_req ? count : num_tokens) * H,
                D >= 128 ? 128 : (D >= 64 ? 64 : 32), 0, stream,
                (const float*)part_o, (const float*)part_ml, p.out, num_splits, H, tile_q0);
    }
    return 0;
  }
  p.heads_per_tile = G < BM ? G : BM;
  p.queries_per_tile = G < BM ? BM / G : 1;
  p.head_tiles = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  const long long gy = (long long)Hkv * p.head_tiles;
  TS_REQUIRE(gy <= 65535, "paged_attention_mma: too many head tiles");
  const size_t smem = (size_t)(BM + 4 * BN) * ROW_BYTES;
  static bool configured_prefill = false;
  if (!configured_prefill) {
    e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("paged_attention_mma: %s", cudaGetErrorString(e));
    configured_prefill = true;
  }
  dim3 grid((max_q_len + p.queries_per_tile - 1) / p.queries_per_tile, (unsigned)gy, num_requests);
  TS_REQUIRE(p.tile_req == nullptr || tile_queries == p.queries_per_tile,
             "paged_attention_mma: the work list was cut for %d queries a block, the kernel takes %d",
             tile_queries, p.queries_per_tile);
  if (p.tile_req) grid = dim3(num_tiles, (unsigned)gy, 1);
  TS_LAUNCH("attn_prefill", attn_prefill_kernel, grid, PRE_THREADS, smem, stream, p);
  return 0;
}
}  // namespace

