// out[M, N] = x[M, K] * W[N, K]^T for many tokens (prompt portions: M from 65 to thousands),
// bfloat16 operands, 32-bit accumulation, on the 5th-generation tensor cores with pairs of SMs.
//
// Two blocks on neighbouring SMs (a cluster of 2) share one tile of 256 tokens x 256 weight rows:
// tcgen05.mma.cta_group::2 reads 128 token rows (A) and 128 weight rows (half of B) from each
// block's shared memory and leaves 128 x 256 accumulators in each block's tensor memory, so every
// SM loads and reads only half of the weight tile.  Per 64-wide slice of K each block's loader
// thread issues two TMA loads (128-byte swizzle, no multicast) into a ring of six stages; both
// blocks' loads complete on the first block's mbarrier.  Four threads of the first block issue
// the four K steps of a stage (one thread issues a tcgen05.mma every 196 cycles at most, measured,
// and an MMA of this size takes 128), all into the same accumulator, and commit the stage back to
// both loaders.  Accumulators are double buffered (2 x 256 of the 512 columns): four epilogue
// warps per block drain tile i (one thread per token row) while tile i + 1 is multiplied, zero
// what they drained (every MMA accumulates, so no order among the issuing threads is needed) and
// hand the buffer back.
//
// The grid is persistent: at most one pair per two SMs.  Whole waves of tiles are dealt round
// robin (neighbouring pairs work on tiles that share their weight rows, which the L2 then serves);
// the tiles of the last, partial wave are cut along K so that all pairs end together.  A pair
// that holds part of such a tile stores its 32-bit partial tile and bumps the tile's counter; the
// block that arrives last adds the parts in order and runs the epilogue.  Nobody waits for anybody.
// (The four issuing threads add into one accumulator in the order in which the tensor core takes
// their instructions, which is not fixed: two runs agree to the rounding of a 32-bit sum.)
//
// Epilogues: plain (optional bias, optional RMSNorm factor per token row), gated (weight rows
// alternate in blocks of 64, gate then up: out = act(gate) * up), residual (residual += result in
// 32-bit; rows residual * norm_weight in bfloat16 and their sums of squares for the next product).
//
// Every mbarrier wait is bounded; a block that gives up raises the library's error flag and the
// engine's status word, tells its partner, stores nothing more and frees its tensor memory.
// tinyserve leaves these products to cuBLAS (serve.py:847, 883, 916, 919, 1263).
#include "tcgen05.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

using bf16 = __nv_bfloat16;
constexpr int BM = 128;              // token rows of a block (256 of the pair)
constexpr int BN = 256;              // weight rows of a tile (128 in each block's shared memory)
constexpr int BK = 64;               // K elements of a stage: 128 bytes, one swizzle row
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ISSUERS = BK / 16;     // one issuing thread per K step of a stage
constexpr int EPI_WARPS = 4;         // warp w reads tensor-memory lanes 32 w .. 32 w + 31
constexpr int LOAD_WARP = EPI_WARPS, ISSUE_WARP0 = EPI_WARPS + 1;
constexpr int THREADS = 32 * (EPI_WARPS + 1 + ISSUERS);
constexpr int TMEM_COLS = 2 * BN;
constexpr int CHUNK = 32, CHUNKS = BN / CHUNK;
constexpr int MIN_TAIL_SLICES = 8;   // a pair takes at least this many K slices of the last wave
constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;

struct PairParams {
  void* out;              // [M, ldc] bfloat16 or float (null in the residual form)
  long long ldc;
  int out_f32;
  int M, N, K;
  int tiles_m, slices;    // tiles along the tokens; 64-wide slices of K
  int pairs;
  int dp_tiles;           // tiles of whole waves, dealt round robin
  int tail_tiles, tail_per, tail_pairs;      // last wave: tail_per slices per pair
  int max_parts;
  float* scratch;         // [tail tile][max_parts][2][CHUNKS][128][32]
  int* counters;          // [tail tile][2], zero between calls
  const float* x_sumsq;   // [x_tiles][x_stride]: sums of squares of the rows of x before their norm
  int x_tiles, x_stride;
  float x_eps;
  VecParam bias;
  int gated_act;          // 0: off, else activation code + 1; out [M, N / 2]
  float* residual;        // [M, N] float, contiguous
  VecParam norm_w;
  bf16* hprime;           // [M, N]
  float* sumsq_out;       // [N / 128 rounded up][sumsq_stride]
  int sumsq_stride;
};

struct Segment {
  int tile, s0, s1;       // K slices [s0, s1) of the tile
  int parts, part, slot;  // parts > 1: a tile of the last wave, this is part `part` of tail tile `slot`
};

// the i-th piece of work of a pair; false when there is none
__device__ __forceinline__ bool segment_of(const PairParams& p, int pair, int i, Segment& s) {
  const int n_dp = pair < p.dp_tiles ? (p.dp_tiles - pair + p.pairs - 1) / p.pairs : 0;
  if (i < n_dp) {
    s.tile = pair + i * p.pairs; s.s0 = 0; s.s1 = p.slices; s.parts = 1; s.part = 0; s.slot = 0;
    return true;
  }
  if (pair >= p.tail_pairs) return false;
  const int total = p.tail_tiles * p.slices;
  const int u0 = pair * p.tail_per, u1 = min(total, u0 + p.tail_per);
  const int t = u0 / p.slices + (i - n_dp);
  const int begin = max(u0, t * p.slices), end = min(u1, (t + 1) * p.slices);
  if (begin >= end) return false;
  const int first = (t * p.slices) / p.tail_per;
  const int last = min(p.tail_pairs - 1, ((t + 1) * p.slices - 1) / p.tail_per);
  s.tile = p.dp_tiles + t; s.s0 = begin - t * p.slices; s.s1 = end - t * p.slices;
  s.parts = last - first + 1; s.part = pair - first; s.slot = t;
  return true;
}

__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// a TMA load of this block's shared memory whose bytes are counted on an mbarrier of either block
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
// one MMA over the pair: D (both blocks' tensor memory) += A (128 rows of each block) * B (128 rows of each block)^T
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(1u) : "memory");
}
// arrives on the mbarrier at this shared-memory offset in both blocks once this thread's MMAs are done
__device__ __forceinline__ void commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;\n" ::"n"(EPI_WARPS * 32) : "memory"); }
// true if `ok` holds for every thread of the epilogue warps (they meet at barrier 1)
__device__ __forceinline__ bool epi_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r) : "r"((uint32_t)ok), "n"(EPI_WARPS * 32) : "memory");
  return r != 0;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, PairParams p) {
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* ctrl = smem + (size_t)STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctrl);            // [STAGES], used in the first block
  uint64_t* empty = full + STAGES;                               // [STAGES], in both blocks
  uint64_t* acc_full = empty + STAGES;                           // [2], in both blocks
  uint64_t* acc_empty = acc_full + 2;                            // [2], used in the first block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* is_last = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                          // 0: the block that issues the MMAs
  const int pair = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), ISSUERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), ISSUERS);
      mbar_init(smem_u32(&acc_empty[b]), 2 * EPI_WARPS);
    }
    *abort_flag = 0;
    *is_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == LOAD_WARP) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  // both blocks' barriers exist before either block's loads or commits may reach them
  cluster_arrive();
  cluster_wait();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();

  auto tell_partner = [&]() {
    const uint32_t remote = map_to_rank(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;\n" ::"r"(remote), "r"(1u) : "memory");
  };

  if (warp == LOAD_WARP) {
    if (lane == 0) {
      const uint32_t full0 = map_to_rank(smem_u32(full), 0);     // the first block's barriers
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Segment sg;
      for (int i = 0; ok && segment_of(p, pair, i, sg); ++i) {
        const int row_x = (sg.tile % p.tiles_m) * 2 * BM + (int)rank * BM;
        const int row_w = (sg.tile / p.tiles_m) * BN + (int)rank * (BN / 2);
        for (int s = sg.s0; s < sg.s1; ++s) {
          ok = mbar_wait(smem_u32(&empty[stage]), phase ^ 1u, abort_flag);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(smem_u32(&full[stage]), 2 * STAGE_BYTES);
          const uint32_t dst = smem_u32(smem + (size_t)stage * STAGE_BYTES);
          tma_load_2d_pair(dst, &map_x, full0 + stage * 8, s * BK, row_x);
          tma_load_2d_pair(dst + A_BYTES, &map_w, full0 + stage * 8, s * BK, row_w);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) tell_partner();
    }
  } else if (warp >= ISSUE_WARP0) {
    if (lane == 0 && rank == 0) {
      const int k_step = warp - ISSUE_WARP0;
      // bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair, N = 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Segment sg;
      for (int i = 0; ok && segment_of(p, pair, i, sg); ++i) {
        const int buf = i & 1;
        ok = mbar_wait(smem_u32(&acc_empty[buf]), (uint32_t)(i >> 1) & 1u, abort_flag);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        for (int s = sg.s0; s < sg.s1; ++s) {
          ok = mbar_spin_wait(smem_u32(&full[stage]), phase, abort_flag);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a = smem_u32(smem + (size_t)stage * STAGE_BYTES);
          umma_pair(d, smem_desc(a) + ((k_step * 32) >> 4), smem_desc(a + A_BYTES) + ((k_step * 32) >> 4), idesc);
          commit_pair(smem_u32(&empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) commit_pair(smem_u32(&acc_full[buf]));
      }
      if (!ok) tell_partner();
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t acc_empty0 = map_to_rank(smem_u32(acc_empty), 0);
    const int r_in = warp * 32 + lane;                            // row of this thread in the block's 128
    float zeros[CHUNK];
#pragma unroll
    for (int e = 0; e < CHUNK; ++e) zeros[e] = 0.f;
    for (int c = 0; c < 2 * CHUNKS; ++c) tmem_store32(lane_addr + c * CHUNK, zeros);
    tmem_store_wait();
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive_cluster(acc_empty0);
      mbar_arrive_cluster(acc_empty0 + 8);
    }

    bool ok = true;
    Segment sg;
    for (int i = 0; ok && segment_of(p, pair, i, sg); ++i) {
      const int buf = i & 1;
      const int tm = sg.tile % p.tiles_m, tn = sg.tile / p.tiles_m;
      const int row = tm * 2 * BM + (int)rank * BM + r_in;
      const bool row_ok = row < p.M;
      const int col0 = tn * BN;
      // (all four warps go on or none does: they meet at barriers below)
      ok = epi_all(mbar_wait(smem_u32(&acc_full[buf]), (uint32_t)(i >> 1) & 1u, abort_flag));
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t acc = lane_addr + buf * BN;
      const bool partial = sg.parts > 1;
      bool finish = true;           // this block runs the tile's epilogue
      float* mine = nullptr;
      if (partial) {
        // the 32-bit partial tile goes to scratch; the tensor memory is free again at once
        mine = p.scratch + ((((size_t)sg.slot * p.max_parts + sg.part) * 2 + rank) * CHUNKS) * (BM * CHUNK);
        for (int c = 0; c < CHUNKS; ++c) {
          float v[CHUNK];
          tmem_load32(acc + c * CHUNK, v);
          tmem_store32(acc + c * CHUNK, zeros);
          float4* dst = reinterpret_cast<float4*>(mine + ((size_t)c * BM + r_in) * CHUNK);
#pragma unroll
          for (int e = 0; e < CHUNK; e += 4) __stcg(dst + e / 4, make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]));
        }
        tmem_store_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8);
        __threadfence();
        epi_barrier();
        if (threadIdx.x == 0) {
          int* counter = p.counters + sg.slot * 2 + rank;
          const int seen = atomicAdd(counter, 1);
          *is_last = seen == sg.parts - 1;
          if (seen == sg.parts - 1) *counter = 0;                 // for the next call
        }
        epi_barrier();
        finish = *is_last != 0;
        epi_barrier();                                            // is_last may be written again
        if (finish) __threadfence();
      }
      if (finish) {
        // the RMSNorm factor of this token row, where x came without it
        float row_scale = 1.f;
        if (p.x_sumsq != nullptr && row_ok) {
          float ss = 0.f;
          for (int t = 0; t < p.x_tiles; ++t) ss += __ldcg(p.x_sumsq + (size_t)t * p.x_stride + row);
          row_scale = rsqrtf(ss / (float)p.K + p.x_eps);
        }
        const float* parts0 = p.scratch + (((size_t)sg.slot * p.max_parts) * 2 + rank) * CHUNKS * (BM * CHUNK);
        // 32 accumulators of chunk c of this thread's row: from tensor memory, or the parts added in order
        auto load_chunk = [&](int c, float (&v)[CHUNK]) {
          if (!partial) {
            tmem_load32(acc + c * CHUNK, v);
            tmem_store32(acc + c * CHUNK, zeros);
            return;
          }
#pragma unroll
          for (int e = 0; e < CHUNK; ++e) v[e] = 0.f;
          for (int q = 0; q < sg.parts; ++q) {
            const float4* src = reinterpret_cast<const float4*>(
                parts0 + (size_t)q * 2 * CHUNKS * (BM * CHUNK) + ((size_t)c * BM + r_in) * CHUNK);
#pragma unroll
            for (int e = 0; e < CHUNK; e += 4) {
              const float4 t = __ldcg(src + e / 4);
              v[e] += t.x; v[e + 1] += t.y; v[e + 2] += t.z; v[e + 3] += t.w;
            }
          }
        };
        if (p.residual != nullptr) {
          float ss = 0.f;
          for (int c = 0; c < CHUNKS; ++c) {
            float v[CHUNK];
            load_chunk(c, v);
            const int col = col0 + c * CHUNK;
            if (row_ok) {
              float* res = p.residual + (size_t)row * p.N + col;
              bf16* hp = p.hprime + (size_t)row * p.N + col;
#pragma unroll
              for (int e = 0; e < CHUNK; e += 8) {
                if (col + e < p.N) {
                  const float4 r0 = *reinterpret_cast<const float4*>(res + e), r1 = *reinterpret_cast<const float4*>(res + e + 4);
                  const float r[8] = {r0.x + v[e], r0.y + v[e + 1], r0.z + v[e + 2], r0.w + v[e + 3],
                                      r1.x + v[e + 4], r1.y + v[e + 5], r1.z + v[e + 6], r1.w + v[e + 7]};
                  *reinterpret_cast<float4*>(res + e) = make_float4(r[0], r[1], r[2], r[3]);
                  *reinterpret_cast<float4*>(res + e + 4) = make_float4(r[4], r[5], r[6], r[7]);
                  float h[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    ss = fmaf(r[j], r[j], ss);
                    h[j] = r[j] * p.norm_w[col + e + j];
                  }
                  *reinterpret_cast<uint4*>(hp + e) = make_uint4(pack2(h[0], h[1]), pack2(h[2], h[3]), pack2(h[4], h[5]), pack2(h[6], h[7]));
                }
              }
            }
            if ((c & 3) == 3) {
              // one sum per 128 columns
              const int t128 = (col0 >> 7) + (c >> 2);
              if (row_ok && t128 * 128 < p.N) p.sumsq_out[(size_t)t128 * p.sumsq_stride + row] = ss;
              ss = 0.f;
            }
          }
        } else if (p.gated_act != 0) {
          const int act = p.gated_act - 1;
          bf16* out = static_cast<bf16*>(p.out);
          for (int h = 0; h < 2; ++h) {
            float g[2][CHUNK], u[2][CHUNK];
            // gate chunks first, then up: the order in which tensor memory is freed does not matter
            load_chunk(h * 4, g[0]);
            load_chunk(h * 4 + 1, g[1]);
            load_chunk(h * 4 + 2, u[0]);
            load_chunk(h * 4 + 3, u[1]);
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              const int ocol = tn * (BN / 2) + h * 64 + sub * CHUNK;
              if (row_ok) {
                bf16* dst = out + (size_t)row * p.ldc + ocol;
#pragma unroll
                for (int e = 0; e < CHUNK; e += 8) {
                  if (ocol + e < p.N / 2) {
                    float o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = activate(g[sub][e + j] * row_scale, act) * (u[sub][e + j] * row_scale);
                    *reinterpret_cast<uint4*>(dst + e) = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
                  }
                }
              }
            }
          }
        } else {
          for (int c = 0; c < CHUNKS; ++c) {
            float v[CHUNK];
            load_chunk(c, v);
            const int col = col0 + c * CHUNK;
            if (row_ok) {
#pragma unroll
              for (int e = 0; e < CHUNK; e += 8) {
                if (col + e < p.N) {
                  float o[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    o[j] = v[e + j] * row_scale;
                    if (p.bias.ptr != nullptr) o[j] += p.bias[col + e + j];
                  }
                  if (p.out_f32) {
                    float* dst = static_cast<float*>(p.out) + (size_t)row * p.ldc + col + e;
                    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
                  } else {
                    bf16* dst = static_cast<bf16*>(p.out) + (size_t)row * p.ldc + col + e;
                    *reinterpret_cast<uint4*>(dst) = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
                  }
                }
              }
            }
          }
        }
        if (!partial) {
          tmem_store_wait();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8);
        }
      }
    }
    if (!ok && lane == 0) tell_partner();
  }
  // neither block leaves (or frees its tensor memory) while the other may still reach its barriers
  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == LOAD_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

bool make_map(CUtensorMap* map, const void* base, int rows, int K, long long ld) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// how the tiles of a product are dealt to `pairs` pairs of blocks
void plan(PairParams& p, int pairs) {
  p.tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles = p.tiles_m * ((p.N + BN - 1) / BN);
  p.slices = (p.K + BK - 1) / BK;
  p.pairs = pairs < tiles ? pairs : tiles;
  if (p.pairs < 1) p.pairs = 1;
  p.dp_tiles = tiles / p.pairs * p.pairs;
  p.tail_tiles = tiles - p.dp_tiles;
  p.tail_per = 0; p.tail_pairs = 0; p.max_parts = 1;
  if (p.tail_tiles > 0) {
    const int total = p.tail_tiles * p.slices;
    p.tail_per = (total + p.pairs - 1) / p.pairs;
    if (p.tail_per < MIN_TAIL_SLICES) p.tail_per = MIN_TAIL_SLICES;
    if (p.tail_per > p.slices) p.tail_per = p.slices;            // (tail_tiles < pairs: never more than a tile)
    p.tail_pairs = (total + p.tail_per - 1) / p.tail_per;
    p.max_parts = (p.slices + p.tail_per - 1) / p.tail_per + 1;
  }
}

}  // namespace

// 1 if a block ever gave up on a wait since the library was loaded (reads device memory: syncs)
TS_EXPORT int ts_gemm_pair_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_error_flag, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// pairs of blocks that can be resident at once on this device (0 if the query fails)
TS_EXPORT int ts_gemm_pair_max_pairs() {
  if (cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel, &cfg) != cudaSuccess) return 0;
  return clusters;
}

// scratch floats and counters (ints) that a product of this size needs with `pairs` pairs of blocks
TS_EXPORT long long ts_gemm_pair_scratch(int M, int N, int K, int pairs, int* counters_needed) {
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  plan(p, pairs);
  if (counters_needed) *counters_needed = p.tail_tiles * 2;
  return (long long)p.tail_tiles * p.max_parts * 2 * BM * BN;
}

// x [M, K] (leading dimension ldx), w [N, K] (ldw), bfloat16; out [M, ldc] bfloat16 or float.
// pairs: pairs of blocks to launch (half the SMs, or fewer).  scratch / counters: as
// ts_gemm_pair_scratch says; the counters all zero (the kernel returns them to zero).
// bias [N] (float or bfloat16): added to every row, plain form only.
// x_sumsq [x_tiles][x_stride] != nullptr: the rows of x lack their RMSNorm factor; row m of the
// result is scaled by rsqrt(sum_t x_sumsq[t][m] / K + x_eps) (plain and gated forms).
// gated_act != 0: the rows of w alternate in blocks of 64, gate rows then the matching up rows;
// out [M, N / 2] bfloat16 = act(gate) * up with act = gated_act - 1 (0 SiLU, 1 GELU-tanh); N a multiple of 128.
// residual != nullptr (out unused): residual [M, N] (float, contiguous) += x w^T; hprime [M, N]
// (bfloat16) = residual * norm_w; sumsq_out [N / 128 rounded up][sumsq_stride >= M] = the sums of
// residual^2 over each 128 columns.
TS_EXPORT int ts_gemm_pair(const void* x, const void* w, void* out, int M, int N, int K, long long ldx, long long ldw,
                           long long ldc, int out_f32, const void* bias, int bias_is_f32, const float* x_sumsq,
                           int x_tiles, int x_stride, float x_eps, int gated_act, float* residual,
                           const void* norm_w, int norm_w_is_f32, void* hprime, float* sumsq_out, int sumsq_stride,
                           float* scratch, long long scratch_floats, int* counters, int num_counters, int pairs,
                           cudaStream_t stream) {
  TS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_pair: empty operand");
  TS_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && N % 8 == 0,
             "gemm_pair: N, K and the leading dimensions must be multiples of 8, got N=%d K=%d", N, K);
  TS_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
             "gemm_pair: operands must be 16-byte aligned");
  TS_REQUIRE(pairs >= 1 && pairs <= 1024, "gemm_pair: pairs out of range");
  TS_REQUIRE(residual != nullptr || (out != nullptr && ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0),
             "gemm_pair: the output must be 16-byte aligned with a leading dimension that is a multiple of 8");
  TS_REQUIRE(gated_act == 0 || (gated_act <= 2 && !out_f32 && residual == nullptr && bias == nullptr && N % 128 == 0),
             "gemm_pair: the gated form takes a bfloat16 output, no bias and whole blocks of 64 gate and 64 up rows");
  TS_REQUIRE(residual == nullptr || (norm_w && hprime && sumsq_out && sumsq_stride >= M && bias == nullptr && x_sumsq == nullptr
                                     && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 && (reinterpret_cast<uintptr_t>(hprime) & 15) == 0),
             "gemm_pair: the residual form needs the norm's weight, both outputs (16-byte aligned) and a stride of at least M");
  TS_REQUIRE(x_sumsq == nullptr || (x_tiles > 0 && x_stride >= M), "gemm_pair: sums of squares without their tile count or stride");
  PairParams p;
  p.out = out; p.ldc = ldc; p.out_f32 = out_f32;
  p.M = M; p.N = N; p.K = K;
  plan(p, pairs);
  const long long need = (long long)p.tail_tiles * p.max_parts * 2 * BM * BN;
  TS_REQUIRE(p.tail_tiles == 0 || (scratch && counters && scratch_floats >= need && num_counters >= 2 * p.tail_tiles),
             "gemm_pair: %lld floats of scratch and %d counters are needed", need, 2 * p.tail_tiles);
  p.scratch = scratch; p.counters = counters;
  p.x_sumsq = x_sumsq; p.x_tiles = x_tiles; p.x_stride = x_stride; p.x_eps = x_eps;
  p.bias = VecParam{bias, bias_is_f32};
  p.gated_act = gated_act;
  p.residual = residual; p.norm_w = VecParam{norm_w, norm_w_is_f32};
  p.hprime = static_cast<bf16*>(hprime); p.sumsq_out = sumsq_out; p.sumsq_stride = sumsq_stride;
  CUtensorMap mx, mw;
  TS_REQUIRE(make_map(&mx, x, M, K, ldx), "gemm_pair: cuTensorMapEncodeTiled failed for the activations");
  TS_REQUIRE(make_map(&mw, w, N, K, ldw), "gemm_pair: cuTensorMapEncodeTiled failed for the weights");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return ts_fail("gemm_pair: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaError_t e = ts_launch_cluster(gemm_pair_kernel, dim3(2 * p.pairs), dim3(THREADS), SMEM, stream, dim3(2, 1, 1), mx, mw, p);
  if (e != cudaSuccess) return ts_fail("gemm_pair (%d pairs): %s", p.pairs, cudaGetErrorString(e));
  return 0;
}
