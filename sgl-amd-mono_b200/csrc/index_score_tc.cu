// Index scores on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// score[t, c] = sum_h w[t,h] * relu( sum_g 2^(qe[h,g] + ke[c,g]) * sum_{d in group g} q[h,d] k[c,d] )
//
// One tile is 128 keys (two 64-slot index pages of the row's request) x 64 heads, computed as two sub-tiles of
// 32 heads.  Every E2M1 code is exact in e4m3, so a CTA expands the tile's packed FP4 keys once into shared
// memory in the canonical K-major no-swizzle operand layout ([16-byte k chunk][row][16 B]) and issues, per
// sub-tile, four M128 N32 K32 kind::f8f6f4 MMAs, one per 32-dim scale group, each into its own 32-column
// accumulator in tensor memory: the group sums come out exact and the two power-of-two scales are applied in
// the epilogue.  In the epilogue a thread owns one key
// (= one TMEM lane) and walks the 64 heads in registers, so the head reduction needs no shuffles; it adds the
// heads in a fixed order (pair (i, i+8) of every 16-head tile, tiles in order, then offsets 4, 2, 1) so the
// result is bit-identical to the CPU restatement.
//
// A CTA holds 128 TMEM columns and 26 KB of shared memory; four CTAs share an SM, so that one CTA's MMAs and
// loads overlap the others' epilogues (the epilogue's instruction issue is what bounds the kernel).
// Every wait on the MMA-completion mbarrier is bounded: on timeout the CTA records (site << 16 | cta) in the
// status word, frees its tensor memory and returns.
#include "common.cuh"
#include "launch.h"
#include "tma_ring.cuh"

namespace b200mono {

namespace {

__device__ __forceinline__ uint32_t e2m1x4_to_e4m3x4(uint32_t codes) {
  const uint32_t lut_lo = 0x3c383000u, lut_hi = 0x4c484440u;  // 0, .5, 1, 1.5 | 2, 3, 4, 6 as e4m3
  const uint32_t mag = __byte_perm(lut_lo, lut_hi, codes & 0x7777u);
  const uint32_t s = codes & 0x8888u;
  const uint32_t sign = ((s & 0x8u) << 4) | ((s & 0x80u) << 8) | ((s & 0x800u) << 12) | ((s & 0x8000u) << 16);
  return mag | sign;
}
// 16 bytes of packed codes (32 dims, low nibble = even dim) -> 32 e4m3 bytes in dim order
__device__ __forceinline__ void expand16(const uint4 c, uint4& lo, uint4& hi) {
  lo.x = e2m1x4_to_e4m3x4(c.x & 0xffffu);
  lo.y = e2m1x4_to_e4m3x4(c.x >> 16);
  lo.z = e2m1x4_to_e4m3x4(c.y & 0xffffu);
  lo.w = e2m1x4_to_e4m3x4(c.y >> 16);
  hi.x = e2m1x4_to_e4m3x4(c.z & 0xffffu);
  hi.y = e2m1x4_to_e4m3x4(c.z >> 16);
  hi.z = e2m1x4_to_e4m3x4(c.w & 0xffffu);
  hi.w = e2m1x4_to_e4m3x4(c.w >> 16);
}
__device__ __forceinline__ float e8m0_f32(uint32_t code) {
  return code == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(code << 23);
}

constexpr int kTileKeys = 128;
constexpr int kHeads = 64;
constexpr int kHalfHeads = 32;
constexpr int kMaxLocalTiles = 64;  // tiles one CTA takes at most (the launch sizes the grid accordingly)
constexpr int kTmemCols = 128;  // 4 groups x 32 heads
// instruction descriptor of kind::f8f6f4: D f32 (bit 4), A and B e4m3 K-major, N = 32 (>>3 at bit 17), M = 128 (>>4 at bit 24)
constexpr uint32_t kIdesc = (1u << 4) | ((kHalfHeads >> 3) << 17) | ((kTileKeys >> 4) << 24);

// shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices of 128 contiguous bytes;
// `lbo` = bytes between the two 16-byte k chunks of a K=32 step, `sbo` = bytes between 8-row groups
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u)  // p = false: D = A * B (no accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

constexpr int kRing = 2;                        // raw key tiles in flight (bulk copies)
constexpr int kRawTile = 2 * (4096 + 256);      // two pages' codes and scale codes
constexpr int kMaxRows = 64;

}  // namespace

__global__ __launch_bounds__(128, 4) void index_score_tc_kernel(B200IndexScoreArgs a) {
  pdl_enter();
  __shared__ __align__(128) uint8_t s_keys[8 * kTileKeys * 16];  // MMA operand: [k chunk 8][key 128][16 B]
  __shared__ __align__(128) uint8_t s_q[8 * kHeads * 16];        // MMA operand: [k chunk 8][head 64][16 B]
  __shared__ __align__(128) uint8_t s_raw[kRing][kRawTile];      // as in the cache: page 0 codes | page 1 codes | scales 0 | scales 1
  __shared__ __align__(16) float s_qs[kHeads][4];                 // 2^(qe - 127) per head and group
  __shared__ float s_w[kHeads];
  __shared__ __align__(8) uint64_t s_bar, s_full[kRing];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_cum[kMaxRows + 1], s_ctx[kMaxRows], s_req[kMaxRows];
  // this CTA's tiles: row, tile of the row, and the physical pages of the tile's two halves
  __shared__ int s_trow[kMaxLocalTiles], s_ttile[kMaxLocalTiles], s_tpage[kMaxLocalTiles][2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // plan: one round of loads for the rows' key counts, one for the pages of this CTA's tiles
  if (warp == 0) {
    int run = 0;
    for (int t0 = 0; t0 < a.rows; t0 += 32) {
      const int t = t0 + lane;
      const int n = t < a.rows ? a.ctx_len[t] : 0;
      if (t < a.rows) {
        s_ctx[t] = n;
        s_req[t] = a.req_of_row[t];
      }
      int tiles = (n + kTileKeys - 1) / kTileKeys, inc = tiles;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += v;
      }
      if (t < a.rows) s_cum[t + 1] = run + inc;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) s_cum[0] = 0;
  }
  if (tid == 0) {
    mbar_init(&s_bar, 1);
    for (int i = 0; i < kRing; ++i) mbar_init(&s_full[i], 1);
    mbar_fence_init();
    s_abort = 0;
  }
  __syncthreads();
  const int total_tiles = s_cum[a.rows];
  const int per = (total_tiles + gridDim.x - 1) / gridDim.x;
  const int first = blockIdx.x * per, last = min(total_tiles, first + per);
  if (first >= last) return;
  const int n_local = last - first;
  for (int i = tid; i < 2 * n_local; i += 128) {
    const int idx = first + (i >> 1);
    int row = 0;
    while (s_cum[row + 1] <= idx) ++row;
    const int tile = idx - s_cum[row];
    const int page = tile * 2 + (i & 1);
    s_tpage[i >> 1][i & 1] = page * 64 < s_ctx[row] ? a.page_table[(size_t)s_req[row] * a.max_pages + page] : -1;
    if ((i & 1) == 0) {
      s_trow[i >> 1] = row;
      s_ttile[i >> 1] = tile;
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
  WaitCtx wctx{&s_abort, a.status};

  const uint8_t* cache = reinterpret_cast<const uint8_t*>(a.idx_cache);
  const uint64_t policy = policy_evict_first();
  // thread 0: bulk copies of a tile's pages into ring slot local % kRing (a missing second page is skipped)
  auto fetch = [&](int local) {
    const int slot = local % kRing;
    const int p0 = s_tpage[local][0], p1 = s_tpage[local][1];
    mbar_arrive_expect_tx(&s_full[slot], p1 >= 0 ? kRawTile : kRawTile / 2);
    bulk_g2s(s_raw[slot], cache + (size_t)p0 * 4352, 4096, &s_full[slot], policy);
    bulk_g2s(s_raw[slot] + 8192, cache + (size_t)p0 * 4352 + 4096, 256, &s_full[slot], policy);
    if (p1 >= 0) {
      bulk_g2s(s_raw[slot] + 4096, cache + (size_t)p1 * 4352, 4096, &s_full[slot], policy);
      bulk_g2s(s_raw[slot] + 8192 + 256, cache + (size_t)p1 * 4352 + 4096, 256, &s_full[slot], policy);
    }
  };
  if (tid == 0)
    for (int l = 0; l < kRing - 1 && l < n_local; ++l) fetch(l);

  // sub-tile = (tile, half of the heads): four K=32 MMAs, one 32-column accumulator per scale group
  auto issue = [&](int half) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t ka = smem_u32(s_keys), qa = smem_u32(s_q) + half * kHalfHeads * 16;
#pragma unroll
    for (int g = 0; g < 4; ++g)
      mma_f8_ss(tmem + g * kHalfHeads, smem_desc(ka + 2 * g * kTileKeys * 16, kTileKeys * 16, 128),
                smem_desc(qa + 2 * g * kHeads * 16, kHeads * 16, 128), kIdesc);
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s_bar))
                 : "memory");
  };

  int q_row = -1;
  uint32_t phase = 0;
  bool ok = true;
  for (int local = 0; ok && local < n_local; ++local) {
    const int row = s_trow[local];
    if (row != q_row) {  // the row's query operand: 64 heads x 128 dims, expanded like the keys
      q_row = row;
      __syncthreads();  // the previous row's epilogue constants are still being read
      const uint8_t* qrec = reinterpret_cast<const uint8_t*>(a.q_rec) + (size_t)row * kHeads * 68;
      for (int i = tid; i < kHeads * 4; i += 128) {
        const int h = i >> 2, g = i & 3;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(qrec + h * 68 + g * 16);  // 68-byte records: 4-byte aligned
        uint4 lo, hi;
        expand16(make_uint4(src[0], src[1], src[2], src[3]), lo, hi);
        *reinterpret_cast<uint4*>(s_q + ((2 * g) * kHeads + h) * 16) = lo;
        *reinterpret_cast<uint4*>(s_q + ((2 * g + 1) * kHeads + h) * 16) = hi;
      }
      if (tid < kHeads) {
        const uint32_t sc = *reinterpret_cast<const uint32_t*>(qrec + tid * 68 + 64);
        *reinterpret_cast<float4*>(s_qs[tid]) = make_float4(e8m0_f32(sc & 0xffu), e8m0_f32((sc >> 8) & 0xffu),
                                                            e8m0_f32((sc >> 16) & 0xffu), e8m0_f32(sc >> 24));
        s_w[tid] = a.w[(size_t)row * kHeads + tid];
      }
    }
    // the tile's packed keys -> operand layout; thread = key; chunk order rotated per lane pair against bank conflicts
    const int slot = local % kRing;
    if (!mbar_wait(&s_full[slot], (uint32_t)(local / kRing) & 1u, wctx, 8)) break;
    const uint8_t* raw = s_raw[slot];
    float ks[4];
    {
      const uint32_t ksc = *reinterpret_cast<const uint32_t*>(raw + 8192 + tid * 4);
#pragma unroll
      for (int g = 0; g < 4; ++g) ks[g] = e8m0_f32((ksc >> (8 * g)) & 0xffu);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int g = (j + (tid >> 1)) & 3;
        uint4 lo, hi;
        expand16(*reinterpret_cast<const uint4*>(raw + tid * 64 + g * 16), lo, hi);
        *reinterpret_cast<uint4*>(s_keys + ((2 * g) * kTileKeys + tid) * 16) = lo;
        *reinterpret_cast<uint4*>(s_keys + ((2 * g + 1) * kTileKeys + tid) * 16) = hi;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA's reads
    float pair[8], held[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) pair[i] = 0.f;
#pragma unroll 1
    for (int half = 0; half < 2 && ok; ++half) {
      // every thread is past the previous epilogue (accumulators) and, for half 0, its operand writes are done
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();
      if (tid == 0) {
        issue(half);
        // ring slot (local + kRing - 1) % kRing was read by the expansion of tile local - 1: free since the sync above
        if (half == 0 && local + kRing - 1 < n_local) fetch(local + kRing - 1);
      }
      if (!mbar_wait(&s_bar, phase, wctx, 7)) {
        ok = false;
        break;
      }
      phase ^= 1u;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // eight heads at a time, the next eight's accumulators already on their way from tensor memory; heads i and
      // i + 8 of a 16-head tile meet in the step pairs (0,1) and (2,3)
      float d[2][4][8];
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld8(lane_base + g * kHalfHeads, d[0][g]);
#pragma unroll
      for (int t8 = 0; t8 < 4; ++t8) {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (t8 + 1 < 4) {
#pragma unroll
          for (int g = 0; g < 4; ++g) tmem_ld8(lane_base + g * kHalfHeads + (t8 + 1) * 8, d[(t8 + 1) & 1][g]);
        }
        float term[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int h = half * kHalfHeads + t8 * 8 + i;
          const float4 qs = *reinterpret_cast<const float4*>(s_qs[h]);
          float acc = __fmul_rn(d[t8 & 1][0][i], __fmul_rn(qs.x, ks[0]));
          acc = __fmaf_rn(d[t8 & 1][1][i], __fmul_rn(qs.y, ks[1]), acc);
          acc = __fmaf_rn(d[t8 & 1][2][i], __fmul_rn(qs.z, ks[2]), acc);
          acc = __fmaf_rn(d[t8 & 1][3][i], __fmul_rn(qs.w, ks[3]), acc);
          term[i] = __fmul_rn(fmaxf(acc, 0.f), s_w[h]);
        }
        if ((t8 & 1) == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) held[i] = term[i];
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) pair[i] = __fadd_rn(pair[i], __fadd_rn(held[i], term[i]));
        }
      }
    }
    if (!ok) break;
    float q4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q4[i] = __fadd_rn(pair[i], pair[i + 4]);
    const float score = __fadd_rn(__fadd_rn(q4[0], q4[2]), __fadd_rn(q4[1], q4[3]));
    const int key = s_ttile[local] * kTileKeys + tid;
    if (key < s_ctx[row]) a.scores[(size_t)row * a.score_stride + key] = score;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

cudaError_t launch_index_score_tc(const B200IndexScoreArgs& a, cudaStream_t s) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // four CTAs of 45 KB per SM: ask for the largest shared-memory carve-out, or only two become resident
    cudaFuncSetAttribute(index_score_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  // the rows' real tile counts are on the device (the CTAs split them evenly); the grid only needs an upper bound
  const int bound = a.rows * ((a.max_ctx + kTileKeys - 1) / kTileKeys);
  int grid = 4 * sms;
  if (grid * kMaxLocalTiles < bound) grid = (bound + kMaxLocalTiles - 1) / kMaxLocalTiles;
  if (grid > bound) grid = bound;
  launch_pdl(index_score_tc_kernel, grid, 128, 0, s, a);
  return cudaGetLastError();
}

}  // namespace b200mono
