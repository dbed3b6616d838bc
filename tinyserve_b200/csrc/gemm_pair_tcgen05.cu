// out[M, N] = x[M, K] * W[N, K]^T for many tokens (prompt portions: M from 65 to thousands),
// bfloat16 operands, 32-bit accumulation, on the 5th-generation tensor cores with pairs of SMs.
//
// Two blocks on neighbouring SMs (a cluster of 2) share one tile of 256 tokens x 256 weight rows
// (or x 512, see Cfg): tcgen05.mma.cta_group::2 reads 128 token rows (A) and 128 weight rows
// (half of B) from each block's shared memory and leaves 128 x 256 accumulators in each block's
// tensor memory, so every SM loads and reads only half of the weight tile.  Per 64-wide slice of
// K each block's loader thread issues its TMA loads (128-byte swizzle, every block its own: no
// cluster-wide copies) into a ring of five stages; both blocks' loads complete on the first
// block's mbarrier.  Four threads of the first block issue
// the four K steps of a stage (one thread issues a tcgen05.mma every 196 cycles at most, measured,
// and an MMA of this size takes 128), all into the same accumulator, and commit the stage back to
// both loaders.  Accumulators are double buffered (2 x 256 of the 512 columns): four epilogue
// warps per block drain tile i (one thread per token row) while tile i + 1 is multiplied, zero
// what they drained (every MMA accumulates, so no order among the issuing threads is needed) and
// hand the buffer back.
//
// The epilogue warps reach global memory through tiles of 128 rows x 128 bytes in shared memory,
// so that a warp's loads and stores cover whole lines; stores are not waited for, and the residual
// rows of the next 32 columns are loaded while these are handled.  (Two other ways were measured
// on a tile of bfloat16 rows: threads storing their own rows, 16 bytes to each of 32 lines per
// instruction, 9 us; TMA stores, which queue behind the loader's TMA loads, 12 us.)
//
// The grid is persistent: at most one pair per two SMs.  Whole waves of tiles are dealt round
// robin (neighbouring pairs work on tiles that share their weight rows, which the L2 then serves);
// the tiles of the last, partial wave are cut along K so that all pairs end together, where that
// pays.  A pair that holds part of such a tile adds its 32-bit partial tile to the tile's sum in
// global memory (red.global.add; in the residual form the sum is the residual itself) and bumps the
// tile's counter; the block that arrives last runs the epilogue on the sum.  Nobody waits for
// anybody.  (The four issuing threads add into one accumulator in the order in which the tensor
// core takes their instructions, and the parts of a cut tile in the order in which they arrive:
// two runs agree to the rounding of a 32-bit sum, not bit by bit.)
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
constexpr int HALF_N = 256;          // weight rows of one MMA over the pair (128 in each block's shared memory)
constexpr int BK = 64;               // K elements of a stage: 128 bytes, one swizzle row
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (HALF_N / 2) * BK * 2;
constexpr int ISSUERS = BK / 16;     // one issuing thread per K step of a stage
constexpr int LOAD_WARP = 4, ISSUE_WARP0 = 5;        // warps 0-3: epilogue; 4: loads; 5-8: issue (and epilogue)
constexpr int THREADS = 32 * (ISSUE_WARP0 + ISSUERS);
constexpr int TMEM_COLS = 512;
constexpr int CHUNK = 32, CHUNKS = HALF_N / CHUNK;
constexpr int TILE_BYTES = BM * 128; // an epilogue tile in shared memory: 128 rows of 128 bytes (32 float or 64 bfloat16)

// HALVES = 1: tiles of 256 x 256, two accumulators in turn: the epilogue of a tile runs beside the
// next tile's MMAs (and is slow there: the MMAs keep the tensor memory busy, a tile takes 9 to 14
// us to drain, which a mainloop of 64 slices of K still hides).  HALVES = 2: tiles of 256 x 512,
// one accumulator of all 512 columns: a block loads 48 KB per eight MMAs instead of 32 KB per
// four (with all SMs loading, the L2 delivers about 80 GB/s to each, which bounds the narrower
// tile), and the epilogue runs while no MMA does, by the issuing warps as well.
template <int HALVES> struct Cfg {
  static constexpr int TILE_N = HALF_N * HALVES;
  static constexpr int STAGE_BYTES = A_BYTES + HALVES * B_BYTES;
  static constexpr int STAGES = HALVES == 1 ? 5 : 4;
  static constexpr int BUFFERS = 2 / HALVES;
  static constexpr int GROUPS = HALVES;            // epilogue groups of four warps, one per half
  static constexpr int EPI_TILES = HALVES == 1 ? 2 : 1;      // tiles of each kind (accumulators in, rows out) per group
  static constexpr int ALL_TILES = 2 * GROUPS * EPI_TILES / HALVES;         // four, or two
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + ALL_TILES * TILE_BYTES + 256;
};

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
  float* scratch;         // [tail tile][2][128][256]: where the parts of a cut tile are added (tiles of 256 rows only); zero between calls
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
// the four warps of epilogue group g meet at barrier 1 + g
__device__ __forceinline__ void epi_barrier(int g) { asm volatile("bar.sync %0, 128;\n" ::"r"(1 + g) : "memory"); }
// true if `ok` holds for every thread of the group
__device__ __forceinline__ bool epi_all(int g, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r) : "r"((uint32_t)ok), "r"(1 + g) : "memory");
  return r != 0;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// An epilogue tile in shared memory is 128 rows of 128 bytes with the 128-byte swizzle of the
// tensor maps: the 16-byte unit u of row r lies at unit u ^ (r & 7).  A thread owns row r; eight
// threads of neighbouring rows touch eight different units, so their accesses do not collide.
__device__ __forceinline__ uint4* tile_unit(char* tile, int r, int u) {
  return reinterpret_cast<uint4*>(tile + r * 128 + ((u ^ (r & 7)) << 4));
}
__device__ __forceinline__ void tile_write_f32(char* tile, int r, const float (&v)[CHUNK]) {
#pragma unroll
  for (int u = 0; u < 8; ++u)
    *tile_unit(tile, r, u) = make_uint4(__float_as_uint(v[4 * u]), __float_as_uint(v[4 * u + 1]),
                                        __float_as_uint(v[4 * u + 2]), __float_as_uint(v[4 * u + 3]));
}
__device__ __forceinline__ void tile_read_f32(char* tile, int r, float (&v)[CHUNK]) {
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const uint4 t = *tile_unit(tile, r, u);
    v[4 * u] = __uint_as_float(t.x); v[4 * u + 1] = __uint_as_float(t.y);
    v[4 * u + 2] = __uint_as_float(t.z); v[4 * u + 3] = __uint_as_float(t.w);
  }
}
// 32 values as bfloat16 into units u0 .. u0 + 3 of row r (half of a 64-column tile)
__device__ __forceinline__ void tile_write_bf16(char* tile, int r, int u0, const float (&v)[CHUNK]) {
#pragma unroll
  for (int u = 0; u < 4; ++u)
    *tile_unit(tile, r, u0 + u) = make_uint4(pack2(v[8 * u], v[8 * u + 1]), pack2(v[8 * u + 2], v[8 * u + 3]),
                                             pack2(v[8 * u + 4], v[8 * u + 5]), pack2(v[8 * u + 6], v[8 * u + 7]));
}

// What the four warps of an epilogue group share: tiles for accumulators on their way from the
// row owners to the threads that reach global memory (`acc`) and for output rows (`ost`).  With
// one tile of each kind the two are the same memory (a form of the epilogue uses one kind).
struct EpiShared {
  char* acc;
  char* ost;
};

// The epilogue of one segment for one half (256 columns) of its tile, by the four warps of group
// g.  A thread owns a token row of the tensor memory (quarter = the 32 lanes its warp may read),
// but global memory is reached in another arrangement, through the tiles in shared memory: thread
// t moves the 16-byte unit t & 7 of rows (t >> 3) + 16 j, j = 0..7, so that a warp's instruction
// covers four whole lines of 128 bytes.  Stores are not waited for; the residual rows of the next
// 32 columns are loaded while these are handled.  Returns false if a wait ran out.
template <int HALVES>
__device__ __forceinline__ bool epilogue_half(const PairParams& p, const Segment& sg, int i, int g, int quarter, int lane,
                                              uint32_t rank, uint32_t tmem_base, uint64_t* acc_full, uint32_t acc_empty0,
                                              const EpiShared& sh, volatile int* abort_flag, int* is_last) {
  using C = Cfg<HALVES>;
  constexpr int NT = C::EPI_TILES;
  const int buf = C::BUFFERS == 2 ? (i & 1) : 0;
  const uint32_t parity = C::BUFFERS == 2 ? ((uint32_t)(i >> 1) & 1u) : ((uint32_t)i & 1u);
  const int r_in = quarter * 32 + lane;                        // the row this thread owns in tensor memory
  const int tm = sg.tile % p.tiles_m, tn = sg.tile / p.tiles_m;
  const int row0 = tm * 2 * BM + (int)rank * BM;               // first row of this block's half of the tile
  const int own_row = row0 + r_in;
  const int col0 = tn * C::TILE_N + g * HALF_N;
  const uint32_t acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * HALF_N + g * HALF_N;
  // the other arrangement: unit u of rows rb + 16 j
  const int u = r_in & 7, rb = r_in >> 3;
  float zeros[CHUNK];
#pragma unroll
  for (int e = 0; e < CHUNK; ++e) zeros[e] = 0.f;
  const bool partial = sg.parts > 1;                           // (tiles of 256 rows only)
  auto acc_tile = [&](int b) { return sh.acc + (b & (NT - 1)) * TILE_BYTES; };
  auto ost_tile = [&](int b) { return sh.ost + (b & (NT - 1)) * TILE_BYTES; };
  // with one tile of a kind its readers are done before it is written again
  auto tile_reused = [&]() { if (NT == 1) epi_barrier(g); };
  // 32-bit rows in global memory that chunk c of this block's tile half corresponds to: the
  // residual, or the sum of a cut tile's parts in scratch ([tail tile][2][128][256], zero between tiles)
  float* sum_base = p.residual != nullptr ? p.residual + (size_t)row0 * p.N + col0
                                          : p.scratch + (size_t)(sg.slot * 2 + (int)rank) * BM * HALF_N;
  const size_t sum_ld = p.residual != nullptr ? (size_t)p.N : (size_t)HALF_N;
  auto rows_ok = [&](int j) { return row0 + rb + 16 * j < p.M; };
  // this thread's units of chunk c of the 32-bit rows, eight loads in flight
  auto fetch = [&](int c, float4 (&a)[8], bool in_residual) {
    const bool col_ok = !in_residual || col0 + c * CHUNK + u * 4 < p.N;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      a[j] = (col_ok && (!in_residual || rows_ok(j)))
                 ? __ldcg(reinterpret_cast<const float4*>(sum_base + (size_t)(rb + 16 * j) * sum_ld + c * CHUNK + u * 4))
                 : make_float4(0.f, 0.f, 0.f, 0.f);
  };
  const bool traced = r_in == 0 && g == 0 && rank == 0 && ((blockIdx.x >> 1) % 24) == 0;
  if (traced) timeline_mark_thread(40, i);
  float4 ahead[8];
  // (the residual rows do not depend on the MMAs: the first chunk is on its way during the wait)
  if (p.residual != nullptr && !partial) fetch(0, ahead, true);
  // (all four warps go on or none does: they meet at barriers below)
  if (!epi_all(g, mbar_wait(smem_u32(&acc_full[buf]), parity, abort_flag))) return false;
  tcgen05_fence_after();
  if (traced) timeline_mark_thread(41, sg.s1 - sg.s0);
  auto release_tmem = [&]() {
    tmem_store_wait();
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8);
  };

  if (partial) {
    // this part is added to the tile's sum (reductions that nobody waits for); the tensor memory
    // is free at once
    for (int c = 0; c < CHUNKS; ++c) {
      float v[CHUNK];
      tmem_load32(acc + c * CHUNK, v);
      tmem_store32(acc + c * CHUNK, zeros);
      tile_write_f32(acc_tile(c), r_in, v);
      epi_barrier(g);
      const bool col_ok = p.residual == nullptr || col0 + c * CHUNK + u * 4 < p.N;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (col_ok && (p.residual == nullptr || rows_ok(j))) {
          const uint4 t = *tile_unit(acc_tile(c), rb + 16 * j, u);
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n"
                       ::"l"(sum_base + (size_t)(rb + 16 * j) * sum_ld + c * CHUNK + u * 4), "f"(__uint_as_float(t.x)),
                         "f"(__uint_as_float(t.y)), "f"(__uint_as_float(t.z)), "f"(__uint_as_float(t.w)) : "memory");
        }
      }
      tile_reused();
    }
    release_tmem();
    if (traced) timeline_mark_thread(42, sg.parts);
    __threadfence();
    epi_barrier(g);
    if (r_in == 0) {
      int* counter = p.counters + sg.slot * 2 + rank;
      const int seen = atomicAdd(counter, 1);
      is_last[g] = seen == sg.parts - 1;
      if (seen == sg.parts - 1) *counter = 0;                   // for the next call
    }
    epi_barrier(g);
    const bool finish = is_last[g] != 0;
    if (traced) timeline_mark_thread(44, finish);
    epi_barrier(g);                                             // is_last may be written again
    if (!finish) return true;
    __threadfence();
    if (p.residual != nullptr) fetch(0, ahead, true);
  }
  // the RMSNorm factor of the row this thread owns, where x came without it
  float row_scale = 1.f;
  if (p.x_sumsq != nullptr && own_row < p.M) {
    float ss = 0.f;
    for (int t = 0; t < p.x_tiles; ++t) ss += __ldcg(p.x_sumsq + (size_t)t * p.x_stride + own_row);
    row_scale = rsqrtf(ss / (float)p.K + p.x_eps);
  }
  // chunk c of the accumulators of the row this thread owns: from tensor memory (zeroed behind),
  // or, for the block that finishes a cut tile, the sum of the parts (through a tile in shared
  // memory; the scratch is zeroed behind).  The four warps meet inside.
  auto take = [&](int c, int stage, float (&v)[CHUNK]) {
    if (!partial) {
      tmem_load32(acc + c * CHUNK, v);
      tmem_store32(acc + c * CHUNK, zeros);
      return;
    }
    float4 a[8];
    fetch(c, a, false);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      *tile_unit(acc_tile(stage), rb + 16 * j, u) = make_uint4(__float_as_uint(a[j].x), __float_as_uint(a[j].y),
                                                               __float_as_uint(a[j].z), __float_as_uint(a[j].w));
      __stcg(reinterpret_cast<float4*>(sum_base + (size_t)(rb + 16 * j) * sum_ld + c * CHUNK + u * 4), make_float4(0.f, 0.f, 0.f, 0.f));
    }
    epi_barrier(g);
    tile_read_f32(acc_tile(stage), r_in, v);
  };
  // an output tile of rows of 128 bytes goes to global memory: unit u of rows rb + 16 j
  auto store_tile = [&](const char* tile, char* out_base, size_t ld_bytes, int cols_left_bytes) {
    if (u * 16 >= cols_left_bytes) return;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (rows_ok(j))
        *reinterpret_cast<uint4*>(out_base + (size_t)(rb + 16 * j) * ld_bytes + u * 16) = *tile_unit(const_cast<char*>(tile), rb + 16 * j, u);
  };

  if (p.residual != nullptr) {
    // residual += accumulators (a cut tile's parts are in the residual already); rows residual *
    // norm_w in bfloat16; sums of squares per 128 columns
    float ss[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) ss[j] = 0.f;
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col0 + c * CHUNK + u * 4;
      float4 cur[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[j] = ahead[j];
      if (c + 1 < CHUNKS) fetch(c + 1, ahead, true);
      if (!partial) {
        float v[CHUNK];
        tmem_load32(acc + c * CHUNK, v);
        tmem_store32(acc + c * CHUNK, zeros);
        tile_write_f32(acc_tile(c), r_in, v);
        epi_barrier(g);
      }
      const bool col_ok = col < p.N;
      float w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = col_ok ? p.norm_w[col + e] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 r = cur[j];
        if (!partial) {
          const uint4 t = *tile_unit(acc_tile(c), rb + 16 * j, u);
          r.x += __uint_as_float(t.x); r.y += __uint_as_float(t.y); r.z += __uint_as_float(t.z); r.w += __uint_as_float(t.w);
        }
        if (col_ok && rows_ok(j)) {
          const size_t at = (size_t)(rb + 16 * j) * p.N + c * CHUNK + u * 4;
          if (!partial) __stcg(reinterpret_cast<float4*>(sum_base + at), r);
          *reinterpret_cast<uint2*>(p.hprime + (size_t)row0 * p.N + col0 + at) = make_uint2(pack2(r.x * w[0], r.y * w[1]), pack2(r.z * w[2], r.w * w[3]));
          ss[j] += r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
        }
      }
      if (!partial) tile_reused();
      if ((c & 3) == 3) {
        // one sum per 128 columns: over the eight threads that share a row
        const int t128 = (col0 >> 7) + (c >> 2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float s = ss[j];
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          if (u == 0 && rows_ok(j) && t128 * 128 < p.N) p.sumsq_out[(size_t)t128 * p.sumsq_stride + row0 + rb + 16 * j] = s;
          ss[j] = 0.f;
        }
      }
    }
  } else if (p.gated_act != 0) {
    // out [M, N / 2] = act(gate) * up: 64 output columns a tile, from gate chunks 4h, 4h + 1 and up chunks 4h + 2, 4h + 3
    const int act = p.gated_act - 1;
    for (int h = 0; h < 2; ++h) {
#pragma unroll 1
      for (int sub = 0; sub < 2; ++sub) {
        float gt[CHUNK], up[CHUNK];
        take(h * 4 + sub, 0, gt);
        take(h * 4 + 2 + sub, 1, up);
#pragma unroll
        for (int e = 0; e < CHUNK; ++e) gt[e] = activate(gt[e] * row_scale, act) * (up[e] * row_scale);
        tile_write_bf16(ost_tile(h), r_in, sub * 4, gt);
        if (partial) epi_barrier(g);                            // the tiles that `take` went through are read
      }
      epi_barrier(g);
      const int ocol = (col0 >> 1) + h * 64;
      store_tile(ost_tile(h), reinterpret_cast<char*>(static_cast<bf16*>(p.out) + (size_t)row0 * p.ldc + ocol), (size_t)p.ldc * 2,
                 (p.N / 2 - ocol) * 2);
      tile_reused();
    }
  } else if (p.out_f32) {
    // (a product with 32-bit output is never cut)
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = col0 + c * CHUNK;
      float v[CHUNK];
      tmem_load32(acc + c * CHUNK, v);
      tmem_store32(acc + c * CHUNK, zeros);
#pragma unroll
      for (int e = 0; e < CHUNK; ++e) {
        v[e] *= row_scale;
        if (p.bias.ptr != nullptr && col + e < p.N) v[e] += p.bias[col + e];
      }
      tile_write_f32(ost_tile(c), r_in, v);
      epi_barrier(g);
      store_tile(ost_tile(c), reinterpret_cast<char*>(static_cast<float*>(p.out) + (size_t)row0 * p.ldc + col), (size_t)p.ldc * 4,
                 (p.N - col) * 4);
      tile_reused();
    }
  } else {
    // bfloat16 rows, 64 columns a tile
    for (int q = 0; q < CHUNKS / 2; ++q) {
      const int col = col0 + q * 64;
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        float v[CHUNK];
        take(2 * q + sub, sub, v);
#pragma unroll
        for (int e = 0; e < CHUNK; ++e) {
          v[e] *= row_scale;
          if (p.bias.ptr != nullptr && col + sub * CHUNK + e < p.N) v[e] += p.bias[col + sub * CHUNK + e];
        }
        tile_write_bf16(ost_tile(q), r_in, sub * 4, v);
      }
      epi_barrier(g);
      store_tile(ost_tile(q), reinterpret_cast<char*>(static_cast<bf16*>(p.out) + (size_t)row0 * p.ldc + col), (size_t)p.ldc * 2,
                 (p.N - col) * 2);
      tile_reused();
    }
  }
  if (!partial) release_tmem();
  if (traced) timeline_mark_thread(45, i);
  return true;
}

template <int HALVES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, PairParams p) {
  using C = Cfg<HALVES>;
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* tiles = smem + (size_t)C::STAGES * C::STAGE_BYTES;       // the epilogue's
  char* ctrl = tiles + C::ALL_TILES * TILE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ctrl);            // [STAGES], used in the first block
  uint64_t* empty = full + C::STAGES;                            // [STAGES], in both blocks
  uint64_t* acc_full = empty + C::STAGES;                        // [2], in both blocks
  uint64_t* acc_empty = acc_full + 2;                            // [2], used in the first block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* is_last = const_cast<int*>(abort_flag) + 1;               // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                          // 0: the block that issues the MMAs
  const int pair = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), ISSUERS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), ISSUERS);
      mbar_init(smem_u32(&acc_empty[b]), 2 * 4 * C::GROUPS);     // every epilogue warp of both blocks
    }
    *abort_flag = 0;
    is_last[0] = is_last[1] = 0;
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
  const uint32_t acc_empty0 = map_to_rank(smem_u32(acc_empty), 0);

  // Every accumulator starts at zero and every MMA accumulates: the warps that will drain a part
  // of the tensor memory zero it now (and behind every chunk they drain) and hand it to the
  // issuing threads.
  const bool drains = warp < 4 || (HALVES == 2 && warp >= ISSUE_WARP0);
  const int group = warp < 4 ? 0 : 1, quarter = warp & 3;
  // group g's tiles: with tiles of 256 rows two of each kind, else one that serves as either
  EpiShared sh;
  sh.acc = tiles + (HALVES == 1 ? 0 : group * TILE_BYTES);
  sh.ost = tiles + (HALVES == 1 ? 2 * TILE_BYTES : group * TILE_BYTES);
  if (drains) {
    float zeros[CHUNK];
#pragma unroll
    for (int e = 0; e < CHUNK; ++e) zeros[e] = 0.f;
    const uint32_t mine = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (HALVES == 2) {
      for (int c = 0; c < CHUNKS; ++c) tmem_store32(mine + group * HALF_N + c * CHUNK, zeros);
    } else {
      for (int c = 0; c < 2 * CHUNKS; ++c) tmem_store32(mine + c * CHUNK, zeros);
    }
    tmem_store_wait();
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive_cluster(acc_empty0);
      if (C::BUFFERS == 2) mbar_arrive_cluster(acc_empty0 + 8);
    }
  }

  if (warp == LOAD_WARP) {
    if (lane == 0) {
      const uint32_t full0 = map_to_rank(smem_u32(full), 0);     // the first block's barriers
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Segment sg;
      for (int i = 0; ok && segment_of(p, pair, i, sg); ++i) {
        const int row_x = (sg.tile % p.tiles_m) * 2 * BM + (int)rank * BM;
        const int row_w = (sg.tile / p.tiles_m) * C::TILE_N + (int)rank * (HALF_N / 2);
        for (int s = sg.s0; s < sg.s1; ++s) {
          ok = mbar_wait(smem_u32(&empty[stage]), phase ^ 1u, abort_flag);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(smem_u32(&full[stage]), 2 * C::STAGE_BYTES);
          const uint32_t dst = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
          tma_load_2d_pair(dst, &map_x, full0 + stage * 8, s * BK, row_x);
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_2d_pair(dst + A_BYTES + h * B_BYTES, &map_w, full0 + stage * 8, s * BK, row_w + h * HALF_N);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) tell_partner();
    }
  } else if (warp >= ISSUE_WARP0) {
    const int k_step = warp - ISSUE_WARP0;
    // bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair, N = 256
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(HALF_N >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    Segment sg;
    for (int i = 0; ok && segment_of(p, pair, i, sg); ++i) {
      if (lane == 0 && rank == 0) {
        const int buf = C::BUFFERS == 2 ? (i & 1) : 0;
        const uint32_t parity = C::BUFFERS == 2 ? ((uint32_t)(i >> 1) & 1u) : ((uint32_t)i & 1u);
        ok = mbar_wait(smem_u32(&acc_empty[buf]), parity, abort_flag);
        tcgen05_fence_after();
        if (k_step == 0 && (pair % 24) == 0) timeline_mark_thread(50, i);
        const uint32_t d = tmem_base + buf * HALF_N;
        for (int s = sg.s0; ok && s < sg.s1; ++s) {
          ok = mbar_spin_wait(smem_u32(&full[stage]), phase, abort_flag);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
          const uint64_t step = (uint64_t)((k_step * 32) >> 4);
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            umma_pair(d + h * HALF_N, smem_desc(a) + step, smem_desc(a + A_BYTES + h * B_BYTES) + step, idesc);
          commit_pair(smem_u32(&empty[stage]));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) commit_pair(smem_u32(&acc_full[buf]));
        if (k_step == 0 && (pair % 24) == 0) timeline_mark_thread(51, sg.s1 - sg.s0);
        if (!ok) tell_partner();
      }
      if (HALVES == 2) {
        // the issuing warps drain the second half of the tile
        __syncwarp();
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (ok) ok = epilogue_half<HALVES>(p, sg, i, 1, quarter, lane, rank, tmem_base, acc_full, acc_empty0, sh, abort_flag, is_last);
      }
    }
  } else {
    bool ok = true;
    Segment sg;
    for (int i = 0; ok && segment_of(p, pair, i, sg); ++i)
      ok = epilogue_half<HALVES>(p, sg, i, 0, quarter, lane, rank, tmem_base, acc_full, acc_empty0, sh, abort_flag, is_last);
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

// What a part of a cut tile costs beside its MMAs, in K slices of the tile's mainloop: the
// partial tile is stored once, and the block that finishes the tile reads every part.
constexpr int PART_COST_SLICES = 5;
constexpr int MAX_PARTS = 4;

// How the tiles of a product are dealt to `pairs` pairs of blocks.  Whole waves round robin; the
// tiles of the last wave either one per pair, or cut along K into runs of tail_per slices that
// the pairs take in turn (a run may span two tiles), whichever ends sooner by the estimate above.
void plan(PairParams& p, int pairs, int halves, bool may_cut) {
  may_cut = may_cut && halves == 1;
  p.tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles = p.tiles_m * ((p.N + halves * HALF_N - 1) / (halves * HALF_N));
  p.slices = (p.K + BK - 1) / BK;
  p.pairs = pairs < 1 ? 1 : pairs;
  p.dp_tiles = tiles / p.pairs * p.pairs;
  p.tail_tiles = tiles - p.dp_tiles;
  p.tail_per = 0; p.tail_pairs = 0; p.max_parts = 1;
  if (p.tail_tiles == 0) return;
  const int total = p.tail_tiles * p.slices;
  int best_per = p.slices, best_cost = p.slices;
  const int floor_per = (p.slices + MAX_PARTS - 2) / (MAX_PARTS - 1);       // so that a tile has at most MAX_PARTS parts
  for (int per = (total + p.pairs - 1) / p.pairs; may_cut && per < p.slices; ++per) {
    if (per < floor_per || per < 4) continue;
    const int parts = (p.slices + per - 1) / per + 1;
    const int cost = per + PART_COST_SLICES * (1 + parts);
    if (cost < best_cost) { best_cost = cost; best_per = per; }
    if (per > best_cost) break;
  }
  p.tail_per = best_per;
  p.tail_pairs = (total + p.tail_per - 1) / p.tail_per;
  p.max_parts = p.tail_per >= p.slices ? 1 : (p.slices + p.tail_per - 1) / p.tail_per + 1;
}

template <int HALVES>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const PairParams& p, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<HALVES>::SMEM);
    if (e != cudaSuccess) return ts_fail("gemm_pair: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int blocks = 2 * (p.pairs < p.dp_tiles + p.tail_pairs ? p.pairs : p.dp_tiles + p.tail_pairs);
  cudaError_t e = ts_launch_cluster(gemm_pair_kernel<HALVES>, dim3(blocks), dim3(THREADS), Cfg<HALVES>::SMEM, stream, dim3(2, 1, 1), mx, mw, p);
  if (e != cudaSuccess) return ts_fail("gemm_pair (%d pairs): %s", p.pairs, cudaGetErrorString(e));
  return 0;
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
  if (cudaFuncSetAttribute(gemm_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<1>::SMEM) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = Cfg<1>::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<1>, &cfg) != cudaSuccess) return 0;
  return clusters;
}

// tiles of 256 (1) or 512 (2) weight rows for this product, by an estimate of both
TS_EXPORT int ts_gemm_pair_halves(int M, int N, int K, int pairs) {
  PairParams a, b;
  a.M = b.M = M; a.N = b.N = N; a.K = b.K = K;
  plan(a, pairs, 1, true);
  plan(b, pairs, 2, false);
  // In units of a thirtieth of a microsecond, from measurements at 2,048 and 4,096 tokens: a slice
  // of K takes 0.40 us with the narrow tile and 0.75 us with the wide one (the MMAs bound both);
  // a launch costs about 3 us, the last epilogue of a pair 2 us with the narrow tile, and every
  // epilogue of the wide tile 6 us in the open.
  auto cost = [&](const PairParams& p, int halves) {
    const double slice = halves == 1 ? 12.0 : 22.5;
    const double waves = (double)(p.dp_tiles / p.pairs) * p.slices;
    const double tail = p.tail_tiles == 0 ? 0.0 : (p.tail_per >= p.slices ? p.slices : p.tail_per + 3.0 * PART_COST_SLICES);
    const double tiles_each = p.dp_tiles / p.pairs + (p.tail_tiles > 0 ? 1 : 0);
    return (waves + tail) * slice + (halves == 2 ? 90.0 + 180.0 * tiles_each : 150.0);
  };
  return cost(b, 2) < cost(a, 1) ? 2 : 1;
}

// scratch floats and counters (ints) that a product of this size needs with `pairs` pairs of
// blocks (none with tiles of 512 rows or a 32-bit output, which are never cut)
TS_EXPORT long long ts_gemm_pair_scratch(int M, int N, int K, int pairs, int halves, int out_f32, int* counters_needed) {
  if (halves != 1 && halves != 2) halves = ts_gemm_pair_halves(M, N, K, pairs);
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  plan(p, pairs, halves, !out_f32);
  if (counters_needed) *counters_needed = p.tail_tiles * 2;
  return p.max_parts > 1 ? (long long)p.tail_tiles * 2 * BM * HALF_N : 0;
}

// x [M, K] (leading dimension ldx), w [N, K] (ldw), bfloat16; out [M, ldc] bfloat16 or float.
// pairs: pairs of blocks to launch (half the SMs, or fewer).  halves: 1 or 2 (tiles of 256 or
// 512 weight rows), 0: chosen here.  scratch / counters: as ts_gemm_pair_scratch says, all zero
// (the kernel returns them to zero).
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
                           int halves, cudaStream_t stream) {
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
                                     && !out_f32 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 && (reinterpret_cast<uintptr_t>(hprime) & 15) == 0),
             "gemm_pair: the residual form needs the norm's weight, both outputs (16-byte aligned) and a stride of at least M");
  TS_REQUIRE(x_sumsq == nullptr || (x_tiles > 0 && x_stride >= M), "gemm_pair: sums of squares without their tile count or stride");
  if (halves != 1 && halves != 2) halves = ts_gemm_pair_halves(M, N, K, pairs);
  PairParams p;
  p.out = out; p.ldc = ldc; p.out_f32 = out_f32;
  p.M = M; p.N = N; p.K = K;
  plan(p, pairs, halves, !out_f32);
  const long long need = p.max_parts > 1 ? (long long)p.tail_tiles * 2 * BM * HALF_N : 0;
  TS_REQUIRE(need == 0 || (scratch && counters && scratch_floats >= need && num_counters >= 2 * p.tail_tiles
                           && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0),
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
  return halves == 2 ? launch<2>(mx, mw, p, stream) : launch<1>(mx, mw, p, stream);
}
