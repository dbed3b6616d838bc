// Paged, variable-length, causal grouped-query attention for prefill on the 5th-generation tensor
// cores, bfloat16, head size 64 or 128 (-DTS_HEAD_DIM).
//
// A block of 320 threads handles two tiles of 128 rows = (query, head of one KV group) pairs of one
// request, tile 1 the queries right after tile 0's, and walks their visible keys in tiles of 128.
// Both query tiles use the same keys and values, and one tile's softmax runs while the tensor core
// works for the other:
//   warp 0   loads: the query tiles once (3-D TMA over [token, head, dim]), then per key tile the K
//            and V pages of the request's block table (2-D TMA boxes of one page x 64 columns,
//            128-byte swizzle), keys and values in rings of two stages each, the keys one tile
//            ahead of the values;
//   warp 1 and the last ISSUERS - 1 warps issue tcgen05.mma: S_g = Q_g K^T into tensor memory, and
//            O_g += P_g V (P_g read from tensor memory, V as an N-contiguous operand) once the
//            probabilities are there; the scores of tile g's next key tile follow its P V at once.
//            A thread can issue one tcgen05.mma per 196 cycles, whatever its size (measured), and
//            the products of a tile's chain (scores -> softmax -> P V -> next scores) lie on the
//            critical path: every product's K steps are therefore dealt to ISSUERS threads of
//            different warps, which walk the products in the same order.  Two hand-overs keep the
//            tensor pipe's order right: the P V steps of a tile must all be issued before the first
//            step of its next scores (which overwrites P), and that first step (it overwrites S)
//            before the other steps of the same scores.  O starts as zeros, so that no P V step
//            is the first one;
//   warps 2-5 (tile 0) and 6-9 (tile 1), one thread per row: read the row of S from tensor memory,
//            mask (key j is visible to the query at position p iff j <= p and, with a window
//            W > 0, j > p - W: serve.py:668-680), online softmax in 32-bit with exp2
//            (tinykernels.py:386-413, 993), write P as bfloat16 over the first columns of S_g,
//            rescale the row of O when its maximum moved; at the end divide O by the row sum and
//            store it.
// Tensor memory: all 512 columns (S_0 / P_0, S_1 / P_1, O_0, O_1), taken before the dependent
// kernel may start, so that no block of a successor can sit on columns that this kernel still needs.
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
constexpr int BM = 128;                      // rows of a query tile
constexpr int BN = 128;                      // keys of a tile
constexpr int GROUPS = 2;                    // query tiles of a block
#ifndef TS_ATTN_ISSUERS
#define TS_ATTN_ISSUERS 3
#endif
constexpr int ISSUERS = TS_ATTN_ISSUERS;     // threads that issue the MMAs of every product
constexpr int SOFTMAX_WARP0 = 2;             // warps 2..9: one thread per row of the two query tiles
constexpr int EXTRA_WARP0 = SOFTMAX_WARP0 + GROUPS * 4;     // warps 10..: issuers 1.. (issuer 0 is warp 1)
constexpr int THREADS = 32 * (EXTRA_WARP0 + ISSUERS - 1);
constexpr int K_STAGES = 2;
constexpr int V_STAGES = 2;
constexpr int DCH = D / 64;                  // 64-column chunks of a head
constexpr int CHUNK_BYTES = 128 * 128;       // 128 rows of 128 bytes
constexpr int Q_BYTES = DCH * CHUNK_BYTES;
constexpr int KV_BYTES = DCH * CHUNK_BYTES;  // one of K or V of a tile
constexpr int TMEM_COLS = 512;               // S_0, S_1: 128 columns each (P_g over the first 64 of S_g); O_0 at 256, O_1 at 384
constexpr size_t SMEM = 1024 + GROUPS * Q_BYTES + (K_STAGES + V_STAGES) * KV_BYTES + 256;

struct TcAttnParams {
  bf16* out;                // [T, H, D]
  const int* block_table;   // [B, max_blocks]
  const int* cu_q;          // [B + 1]
  const int* kv_lens;       // [B]
  const int* tile_req;      // optional work list: request and first query of every block
  const int* tile_q0;
  int H, Hkv, page_shift, page_size, max_blocks;
  int heads_per_tile, queries_per_tile, head_tiles;     // of one query tile
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

// (10 warps take the registers of 12, three per scheduler: 168 registers a thread)
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* Qs = smem;                               // [GROUPS][Q_BYTES]
  char* Ks = Qs + GROUPS * Q_BYTES;              // [K_STAGES][KV_BYTES]
  char* Vs = Ks + K_STAGES * KV_BYTES;           // [V_STAGES][KV_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + V_STAGES * KV_BYTES);
  uint64_t* q_full = bars;                       // 1
  uint64_t* k_full = q_full + 1;                 // [K_STAGES]
  uint64_t* k_empty = k_full + K_STAGES;         // [K_STAGES] both tiles' scores of the stage's keys are computed
  uint64_t* v_full = k_empty + K_STAGES;         // [V_STAGES]
  uint64_t* v_empty = v_full + V_STAGES;         // [V_STAGES] the stage's values are added to both O
  uint64_t* s_full = v_empty + V_STAGES;         // [GROUPS] S_g holds the scores of a key tile
  uint64_t* p_full = s_full + GROUPS;            // [GROUPS] P_g is in tensor memory, O_g is rescaled
  uint64_t* o_ready = p_full + GROUPS;           // [GROUPS] O_g holds the sum over the key tiles so far
  uint64_t* pv_issued = o_ready + GROUPS;        // [GROUPS] every issuer has issued its P V steps of the key tile
  uint64_t* s_first = pv_issued + GROUPS;        // [GROUPS] the first step of the scores (it overwrites S_g) is issued
  uint64_t* o_zeroed = s_first + GROUPS;         // [GROUPS] O_g holds zeros
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_zeroed + GROUPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    // (every issuer commits its own MMAs: what they complete counts ISSUERS arrivals)
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), ISSUERS);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), ISSUERS);
    }
    for (int g = 0; g < GROUPS; ++g) {
      mbar_init(smem_u32(&s_full[g]), ISSUERS);
      mbar_init(smem_u32(&p_full[g]), 4);
      mbar_init(smem_u32(&o_ready[g]), ISSUERS);
      mbar_init(smem_u32(&pv_issued[g]), ISSUERS);
      mbar_init(smem_u32(&s_first[g]), 1);
      mbar_init(smem_u32(&o_zeroed[g]), 4);
    }
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
  const uint32_t tmem_base = *tmem_slot;
  // this block holds all of the SM's tensor memory now: only now may a dependent kernel start
  pdl_trigger();
  pdl_wait();

  // with a work list block x handles entry x; else blocks (tile pair, request) cover max_q_len and
  // exit where a request has fewer queries
  const int QPT = p.queries_per_tile, GT = p.heads_per_tile;
  const int b = p.tile_req ? p.tile_req[blockIdx.x] : blockIdx.z;
  const int kvh = blockIdx.y / p.head_tiles, head_tile = blockIdx.y % p.head_tiles;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = p.tile_req ? p.tile_q0[blockIdx.x]
                            : (gridDim.x - 1 - blockIdx.x) * GROUPS * QPT;     // heavy blocks first
  const int kv_len = p.kv_lens[b];
  const int G = p.H / p.Hkv;
  const int g0 = head_tile * GT;
  const int nq_all = max(0, min(GROUPS * QPT, q_len - q0));
  const int groups = nq_all > QPT ? 2 : 1;       // query tiles of this block that hold queries
  const int pos0 = kv_len - q_len + q0;
  const int j_hi = min(kv_len, pos0 + nq_all);
  const int j_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_tile = j_lo / BN, end_tile = (j_hi + BN - 1) / BN;
  const int n_tiles = nq_all > 0 ? end_tile - first_tile : 0;
  // the timeline build follows one block through its tiles (marks 10.. by the issuer, 20.. by a
  // softmax thread of each query tile, 30 by the loader; the value is the key tile)
  const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;

  if (warp == 0) {
    if (n_tiles > 0) {
      if (lane == 0) {
        // queries: rows (query, head) with the head fastest; one box per 64 columns and query tile
        const uint32_t qbar = smem_u32(q_full);
        mbar_expect_tx(qbar, groups * DCH * 64 * 2 * GT * QPT);
        for (int g = 0; g < groups; ++g)
          for (int c = 0; c < DCH; ++c)
            tma_load_3d(smem_u32(Qs + g * Q_BYTES + c * CHUNK_BYTES), &map_q, qbar, c * 64, kvh * G + g0,
                        q_begin + q0 + g * QPT);
      }
      const int* bt = p.block_table + (size_t)b * p.max_blocks;
      const int pages_per_tile = BN >> p.page_shift;
      // Keys and values have rings of their own, and the keys run one tile ahead: a stage of keys
      // is free as soon as both tiles' scores are computed, long before its values have been used.
      // The boxes of a tile (pages x 64-column chunks) are dealt to the lanes of the warp, so that
      // issuing them takes one box's time; lane 0's arrival carries the tile's byte count, so the
      // stage cannot complete before it.
      auto load = [&](bool keys, int t) -> bool {
        const int stages = keys ? K_STAGES : V_STAGES, s = t % stages;
        const int j0 = (first_tile + t) * BN;
        int ok = 1;
        if (lane == 0)
          ok = mbar_wait(smem_u32(keys ? &k_empty[s] : &v_empty[s]), ((t / stages) & 1) ^ 1, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        const uint32_t bar = smem_u32(keys ? &k_full[s] : &v_full[s]);
        if (lane == 0) mbar_expect_tx(bar, KV_BYTES);
        __syncwarp();
        for (int i = lane; i < pages_per_tile * DCH; i += 32) {
          const int pg = i / DCH, c = i % DCH;
          const int j = j0 + (pg << p.page_shift);
          const int page = j < j_hi ? bt[j >> p.page_shift] : 0;          // past the end: the null page
          const int row = (page * p.Hkv + kvh) << p.page_shift;
          const int off = s * KV_BYTES + c * CHUNK_BYTES + (pg << p.page_shift) * 128;
          if (keys) tma_load_2d(smem_u32(Ks + off), &map_k, bar, c * 64, row);
          else tma_load_2d(smem_u32(Vs + off), &map_v, bar, c * 64, row);
        }
        return true;
      };
      bool ok = load(true, 0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        if (t + 1 < n_tiles) ok = load(true, t + 1);
        if (ok) ok = load(false, t);
        if (traced && lane == 0) timeline_mark_thread(30, t);
      }
    }
  } else if (warp == 1 || warp >= EXTRA_WARP0) {
    if (lane == 0 && n_tiles > 0) {
      // issuer `me` of ISSUERS: its share of the K steps of every product, products in one order
      const int me = warp == 1 ? 0 : warp - EXTRA_WARP0 + 1;
      constexpr uint32_t idesc_qk = make_idesc(BM, BN, false);
      constexpr uint32_t idesc_pv = make_idesc(BM, D, true);
      constexpr int QK_STEPS = D / 16, PV_STEPS = BN / 16;
      const int qk_lo = me * QK_STEPS / ISSUERS, qk_hi = (me + 1) * QK_STEPS / ISSUERS;
      const int pv_lo = me * PV_STEPS / ISSUERS, pv_hi = (me + 1) * PV_STEPS / ISSUERS;
      const uint64_t q_desc = smem_desc(smem_u32(Qs)), k_desc = smem_desc(smem_u32(Ks));
      const uint64_t v_desc = smem_desc_mn(smem_u32(Vs), CHUNK_BYTES);
      // S_g = Q_g K^T of key tile t.  `after_pv`: the P V of tile g's previous key tile read P_g
      // from S_g's columns; all of its steps must be in the pipe before step 0 here.
      auto scores = [&](int g, int t, bool after_pv) -> bool {
        const int s = t % K_STAGES;
        if (!mbar_spin_wait(smem_u32(&k_full[s]), (t / K_STAGES) & 1, abort_flag)) return false;
        if (me == 0) {
          if (after_pv && !mbar_spin_wait(smem_u32(&pv_issued[g]), (t - 1) & 1, abort_flag)) return false;
        } else {
          if (!mbar_spin_wait(smem_u32(&s_first[g]), t & 1, abort_flag)) return false;
        }
        tcgen05_fence_after();
        if (traced && me == 0) timeline_mark_thread(10 + g, t);
        // descriptors: a base made once, plus the operand's offset in 16-byte units (the address is
        // the descriptor's low field; shared memory ends below its range).  An issuing thread is
        // one serial chain of instructions: whatever it computes per MMA delays every MMA.
        const uint64_t qd = q_desc + g * (Q_BYTES >> 4), kd = k_desc + s * (KV_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < QK_STEPS; ++k) {
          if (k < qk_lo || k >= qk_hi) continue;
          const uint64_t off = ((k / 4) * CHUNK_BYTES + (k % 4) * 32) >> 4;
          umma(tmem_base + g * BN, qd + off, kd + off, idesc_qk, k > 0 ? 1u : 0u);
          if (k == 0) {
            // step 0 is in the pipe: the other issuers may add theirs
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&s_first[g]));
          }
        }
        tcgen05_commit(smem_u32(&s_full[g]));
        if (g == groups - 1) tcgen05_commit(smem_u32(&k_empty[s]));
        return true;
      };
      // O_g += P_g V of key tile t
      auto values = [&](int g, int t) -> bool {
        const int s = t % V_STAGES;
        if (!mbar_spin_wait(smem_u32(&v_full[s]), (t / V_STAGES) & 1, abort_flag) ||
            !mbar_spin_wait(smem_u32(&p_full[g]), t & 1, abort_flag))
          return false;
        tcgen05_fence_after();
        if (traced && me == 0) timeline_mark_thread(12 + g, t);
        const uint64_t vd = v_desc + s * (KV_BYTES >> 4);
        const uint32_t o_addr = tmem_base + 2 * BN + g * 128, p_addr = tmem_base + g * BN;
#pragma unroll
        for (int k = 0; k < PV_STEPS; ++k) {
          if (k < pv_lo || k >= pv_hi) continue;
          umma_ts(o_addr, p_addr + k * 8, vd + ((k * 16 * 128) >> 4), idesc_pv, 1u);
        }
        // this issuer's steps are in the pipe (the next scores of the tile wait for all issuers')
        tcgen05_fence_before();
        mbar_arrive(smem_u32(&pv_issued[g]));
        tcgen05_commit(smem_u32(&o_ready[g]));
        if (g == groups - 1) tcgen05_commit(smem_u32(&v_empty[s]));
        return true;
      };
      bool ok = mbar_spin_wait(smem_u32(q_full), 0, abort_flag);
      for (int g = 0; ok && g < groups; ++g) ok = scores(g, 0, false);
      for (int g = 0; ok && g < groups; ++g) ok = mbar_spin_wait(smem_u32(&o_zeroed[g]), 0, abort_flag);
      for (int t = 0; ok && t < n_tiles; ++t)
        for (int g = 0; ok && g < groups; ++g) {
          ok = values(g, t);
          if (ok && t + 1 < n_tiles) ok = scores(g, t + 1, true);
        }
    }
  } else {
    // one thread per row of query tile g
    const int g = (warp - SOFTMAX_WARP0) >> 2;
    if (g < groups && n_tiles > 0) {
      const int q4 = warp & 3;
      const int r = q4 * 32 + lane;
      const int qg = q0 + g * QPT;                       // the tile's first query
      const int nq = min(QPT, q_len - qg);
      const int n_valid = QPT > 1 ? nq * GT : min(GT, G - g0);
      const bool valid = r < n_valid;
      const int qi = QPT > 1 ? r / GT : 0, gg = QPT > 1 ? r % GT : r;
      const int pos = valid ? kv_len - q_len + qg + qi : -1;
      const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
      const uint32_t lane_addr = static_cast<uint32_t>(q4 * 32) << 16;
      const uint32_t tmem_s = tmem_base + g * BN, tmem_o = tmem_base + 2 * BN + g * 128;
      const bool tracer = traced && (threadIdx.x & 127) == 64;
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      {
        // O_g starts as zeros: every P V step then accumulates, whichever issuer's comes first
        float zeros[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) zeros[e] = 0.f;
#pragma unroll
        for (int c = 0; c < D; c += 32) tmem_store32(tmem_o + lane_addr + c, zeros);
        tmem_store_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&o_zeroed[g]));
      }
      for (int t = 0; t < n_tiles; ++t) {
        const int j0 = (first_tile + t) * BN;
        ok = mbar_wait(smem_u32(&s_full[g]), t & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        if (tracer) timeline_mark_thread(20 + 4 * g, t);
        const bool all_visible = j0 + BN - 1 <= pos && j0 >= lo;
        // the whole row of S into registers: four loads in flight, one wait
        float sv[BN];
#pragma unroll
        for (int c = 0; c < BN; c += 32) tmem_load32_nowait(tmem_s + lane_addr + c, sv + c);
        tmem_load_wait();
        if (tracer) timeline_mark_thread(21 + 4 * g, t);
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
        // The reference maximum only moves when the row's maximum has grown by more than 2^8:
        // until then the probabilities are taken against the old reference (at most 256, exact
        // enough in bfloat16 and harmless in the 32-bit sums) and O needs no rescaling; the final
        // division by the row sum, kept against the same reference, gives the same result.
        const float m_cand = fmaxf(m, mx * p.scale_log2);
        const float m_new = (m_cand - m <= 8.f) ? m : m_cand;      // -inf - -inf: moves (to -inf), harmless
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = ex2(m - m_safe);
        // (these scores were computed after the previous key tile's P V of this query tile, in
        // order: P_g has been read and the sum in O_g is complete)
        // probabilities -> tensor memory, bfloat16 pairs over the first 64 columns of S_g: the A
        // operand of O += P V
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < BN; c += 64) {
          float packed[32];
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            const float p0 = ex2(fmaf(sv[c + e], p.scale_log2, -m_safe));        // -inf gives 0
            const float p1 = ex2(fmaf(sv[c + e + 1], p.scale_log2, -m_safe));
            sum4[(e / 2) & 3] += p0 + p1;
            packed[e / 2] = __uint_as_float(pack2(p0, p1));
          }
          tmem_store32(tmem_s + lane_addr + c / 2, packed);
        }
        const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        l = l * alpha + sum;
        m = m_new;
        if (tracer) timeline_mark_thread(22 + 4 * g, t);
        if (t > 0 && !__all_sync(0xffffffffu, alpha == 1.f)) {
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
        tmem_store_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (tracer) timeline_mark_thread(23 + 4 * g, t);
        if (lane == 0) mbar_arrive(smem_u32(&p_full[g]));
      }
      if (ok) {
        ok = mbar_wait(smem_u32(&o_ready[g]), (n_tiles - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tcgen05_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + ((size_t)(q_begin + qg + qi) * p.H + kvh * G + g0 + gg) * D;
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
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

// what the compiler and the driver make of the kernel: registers per thread, most threads per
// block, static and (after the opt-in) most dynamic shared memory; and what a launch asks for
TS_EXPORT int ts_attention_tcgen05_resources(int* out8) {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
  out8[6] = (int)e;
  if (cudaFuncGetAttributes(&a, attn_prefill_tc_kernel) != cudaSuccess) return -1;
  out8[0] = a.numRegs; out8[1] = a.maxThreadsPerBlock; out8[2] = (int)a.sharedSizeBytes;
  out8[3] = a.maxDynamicSharedSizeBytes; out8[4] = THREADS; out8[5] = (int)SMEM; out8[7] = (int)a.localSizeBytes;
  return 0;
}

TS_EXPORT int ts_attention_tcgen05_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// q, out [T, H, D]; caches [num_pages, Hkv, page_size, D]; bfloat16.  tile_req / tile_q0 (optional,
// num_tiles ints each): the request and the first query of every block of tile_queries =
// 2 * (128 / group) queries (two query tiles).
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
  const int per_block = GROUPS * p.queries_per_tile;
  TS_REQUIRE(tile_req == nullptr || tile_queries == per_block,
             "paged_attention_tcgen05: the work list was cut for %d queries a block, the kernel takes %d",
             tile_queries, per_block);
  dim3 grid((max_q_len + per_block - 1) / per_block, (unsigned)gy, num_requests);
  if (tile_req) grid = dim3(num_tiles, (unsigned)gy, 1);
  TS_LAUNCH("attn_prefill_tcgen05", attn_prefill_tc_kernel, grid, THREADS, SMEM, stream, mq, mk, mv, p);
  return 0;
}
