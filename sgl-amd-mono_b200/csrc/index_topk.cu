// Sparse-attention indexer: FP4 x FP4 index scores on the tensor cores and the exact top-k.
//
// score[t, c] = sum_h w[t,h] * relu( sum_g 2^(qe[h,g] + ke[c,g]) * sum_{d in group g} q[h,d] k[c,d] )
// with 64 heads x 128 dims, MXFP4 on both sides (E2M1 codes, one E8M0 scale per 32 dims).  Every E2M1
// value is exact in e4m3, and a 32-dim group is exactly one m16n8k32 MMA step, so the group sums come out
// of the tensor core exact and the two power-of-two scales are applied on the accumulator.  Heads are the
// MMA M dimension (4 tiles of 16), keys the N dimension (8 per MMA).
//
// The top-k is exact: radix select (4 passes of 8 bits) on the order-preserving u32 image of the f32
// score, ties at the threshold resolved towards the lower position, output in ascending position order.
#include "common.cuh"
#include "launch.h"

namespace b200mono {

// four E2M1 codes (16 bits, low nibble first) -> four e4m3 bytes
__device__ __forceinline__ uint32_t e2m1x4_to_e4m3x4(uint32_t codes) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 as e4m3 bytes
  const uint32_t lut_lo = 0x3c383000u, lut_hi = 0x4c484440u;
  const uint32_t mag = __byte_perm(lut_lo, lut_hi, codes & 0x7777u);
  const uint32_t s = codes & 0x8888u;
  const uint32_t sign = ((s & 0x8u) << 4) | ((s & 0x80u) << 8) | ((s & 0x800u) << 12) | ((s & 0x8000u) << 16);
  return mag | sign;
}
__device__ __forceinline__ float e8m0_to_f32(uint32_t code) {
  return code == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(code << 23);  // 2^-127 is subnormal
}

constexpr int kPagesPerWarp = 4;
constexpr int kScoreWarps = 4;

// CTA = 4 warps; blockIdx.y = row, blockIdx.x = group of 16 pages (1024 keys); warp w takes pages 4w..4w+3.
// Slot mapping inside a 32-dim group: MMA k-slot 4c+j <-> dim 8c+j, slot 16+4c+j <-> dim 8c+4+j, on both
// operands, so a lane's operand words are the low / high half of one aligned 4-byte load of packed codes.
__global__ __launch_bounds__(kScoreWarps * 32) void index_score_kernel(B200IndexScoreArgs a) {
  __shared__ __align__(16) uint8_t s_page[kScoreWarps][4352];
  const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int n_keys = a.ctx_len[t];
  const int first_page = (blockIdx.x * kScoreWarps + warp) * kPagesPerWarp;
  if (blockIdx.x * kScoreWarps * kPagesPerWarp * 64 >= n_keys) return;
  const int req = a.req_of_row[t];
  const int* pages = a.page_table + (size_t)req * a.max_pages;

  // query fragments: heads mt*16 + g and + 8, group gk; scales and head weights of those two heads
  const uint8_t* qrec = reinterpret_cast<const uint8_t*>(a.q_rec) + (size_t)t * 64 * 68;
  uint32_t A[4][4][4];
  float qs[4][4][2], wh[4][2];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int h = mt * 16 + g + 8 * r;
      const uint8_t* hr = qrec + h * 68;
      wh[mt][r] = a.w[(size_t)t * 64 + h];
#pragma unroll
      for (int gk = 0; gk < 4; ++gk) {
        const uint32_t packed = *reinterpret_cast<const uint32_t*>(hr + gk * 16 + 4 * c);
        A[mt][gk][r] = e2m1x4_to_e4m3x4(packed & 0xffffu);          // a0 / a1
        A[mt][gk][2 + r] = e2m1x4_to_e4m3x4(packed >> 16);          // a2 / a3
        qs[mt][gk][r] = e8m0_to_f32(hr[64 + gk]);
      }
    }
  }

  uint8_t* sp = s_page[warp];
  for (int pi = first_page; pi < first_page + kPagesPerWarp; ++pi) {
    const int key0 = pi * 64;
    if (key0 >= n_keys) break;
    const uint8_t* page = reinterpret_cast<const uint8_t*>(a.idx_cache) + (size_t)pages[pi] * 4352;
    __syncwarp();
    for (int i = lane; i < 4352 / 16; i += 32) reinterpret_cast<uint4*>(sp)[i] = reinterpret_cast<const uint4*>(page)[i];
    __syncwarp();
#pragma unroll 1
    for (int kt = 0; kt < 8; ++kt) {
      float acc[4][4];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
      const uint8_t* krow = sp + (kt * 8 + g) * 64;             // B operand: key kt*8 + g
      const uint8_t* ksc = sp + 4096 + (kt * 8 + 2 * c) * 4;    // D columns: keys kt*8 + 2c, 2c+1
#pragma unroll
      for (int gk = 0; gk < 4; ++gk) {
        const uint32_t packed = *reinterpret_cast<const uint32_t*>(krow + gk * 16 + 4 * c);
        const uint32_t b0 = e2m1x4_to_e4m3x4(packed & 0xffffu), b1 = e2m1x4_to_e4m3x4(packed >> 16);
        const float k0 = e8m0_to_f32(ksc[gk]), k1 = e8m0_to_f32(ksc[4 + gk]);
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          float d[4] = {0.f, 0.f, 0.f, 0.f};
          mma_e4m3_16x8x32(d, A[mt][gk][0], A[mt][gk][1], A[mt][gk][2], A[mt][gk][3], b0, b1);
          // group sums are exact; scale products are exact powers of two; one rounding per add
          acc[mt][0] = __fadd_rn(acc[mt][0], __fmul_rn(d[0], __fmul_rn(qs[mt][gk][0], k0)));
          acc[mt][1] = __fadd_rn(acc[mt][1], __fmul_rn(d[1], __fmul_rn(qs[mt][gk][0], k1)));
          acc[mt][2] = __fadd_rn(acc[mt][2], __fmul_rn(d[2], __fmul_rn(qs[mt][gk][1], k0)));
          acc[mt][3] = __fadd_rn(acc[mt][3], __fmul_rn(d[3], __fmul_rn(qs[mt][gk][1], k1)));
        }
      }
      // heads: pair (g, g+8), xor tree over g, tiles in order
      float tot[2] = {0.f, 0.f};
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float v = __fadd_rn(__fmul_rn(fmaxf(acc[mt][j], 0.f), wh[mt][0]), __fmul_rn(fmaxf(acc[mt][2 + j], 0.f), wh[mt][1]));
          v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
          v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
          v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
          tot[j] = __fadd_rn(tot[j], v);
        }
      }
      if (g == 0) {
        const int key = key0 + kt * 8 + 2 * c;
        float* out = a.scores + (size_t)t * a.score_stride;
        if (key < n_keys) out[key] = tot[0];
        if (key + 1 < n_keys) out[key + 1] = tot[1];
      }
    }
  }
}

cudaError_t launch_index_score(const B200IndexScoreArgs& a, cudaStream_t s) {
  const int keys_per_cta = kScoreWarps * kPagesPerWarp * 64;
  dim3 grid((a.max_ctx + keys_per_cta - 1) / keys_per_cta, a.rows);
  index_score_kernel<<<grid, kScoreWarps * 32, 0, s>>>(a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ exact top-k
// One CTA of 1024 threads per row.
__global__ __launch_bounds__(1024) void topk_kernel(B200TopkArgs a) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int whist[32][256];  // per-warp histograms: score exponents cluster in a few digits
  __shared__ unsigned int s_prefix, s_need, s_scan[32], s_base_gt, s_base_eq;
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = a.ctx_len[t];
  const float* sc = a.scores + (size_t)t * a.score_stride;
  int* out = a.topk_idx + (size_t)t * a.k;
  if (n <= a.k) {
    for (int i = tid; i < n; i += 1024) out[i] = i;
    if (tid == 0) a.topk_count[t] = n;
    return;
  }
  if (tid == 0) {
    s_prefix = 0;
    s_need = (unsigned)a.k;
  }
  // radix select from the most significant byte: afterwards s_prefix is the k-th largest key and
  // s_need the number of keys equal to it that belong to the top-k
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 32 * 256; i += 1024) (&whist[0][0])[i] = 0;
    __syncthreads();
    const unsigned prefix = s_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i0 = 0; i0 < n; i0 += 1024) {
      const int i = i0 + tid;
      unsigned digit = 256u;  // not a candidate
      if (i < n) {
        const unsigned key = radix_key(sc[i]);
        if ((key & mask) == prefix) digit = (key >> shift) & 0xffu;
      }
      // lanes with the same digit elect one to add their count
      const unsigned peers = __match_any_sync(0xffffffffu, digit);
      if (digit < 256u && lane == __ffs(peers) - 1) whist[warp][digit] += (unsigned)__popc(peers);
      __syncwarp();
    }
    __syncthreads();
    if (tid < 256) {
      unsigned c = 0;
      for (int w = 0; w < 32; ++w) c += whist[w][tid];
      hist[tid] = c;
    }
    __syncthreads();
    if (warp == 0) {
      // digits from high to low: find the digit where the running count reaches s_need
      unsigned need = s_need, run = 0;
      int found = -1;
      for (int base = 224; base >= 0 && found < 0; base -= 32) {
        const unsigned cnt = hist[base + 31 - lane];  // lane 0 holds the highest digit of the block
        unsigned incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl += o;
        }
        const bool hit = run + incl >= need;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (ballot) {
          const int l = __ffs(ballot) - 1;
          const unsigned before = run + __shfl_sync(0xffffffffu, incl, l) - __shfl_sync(0xffffffffu, cnt, l);
          found = base + 31 - l;
          if (lane == 0) {
            s_need = need - before;
            s_prefix = prefix | ((unsigned)found << shift);
          }
        } else {
          run += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
    }
    __syncthreads();
  }
  const unsigned thr = s_prefix, need_eq = s_need;
  if (tid == 0) {
    s_base_gt = 0;
    s_base_eq = 0;
  }
  __syncthreads();
  // emit in ascending position: everything above the threshold, and the first need_eq keys equal to it
  for (int i0 = 0; i0 < n; i0 += 1024) {
    const int i = i0 + tid;
    unsigned key = 0;
    if (i < n) key = radix_key(sc[i]);
    const bool gt = i < n && key > thr, eq = i < n && key == thr;
    const unsigned bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) s_scan[warp] = (unsigned)__popc(bg) | ((unsigned)__popc(be) << 16);
    __syncthreads();
    unsigned before_gt = 0, before_eq = 0, tot_gt = 0, tot_eq = 0;
    for (int w = 0; w < 32; ++w) {
      const unsigned v = s_scan[w];
      if (w < warp) {
        before_gt += v & 0xffffu;
        before_eq += v >> 16;
      }
      tot_gt += v & 0xffffu;
      tot_eq += v >> 16;
    }
    const unsigned lm = (1u << lane) - 1u;
    const unsigned my_gt = s_base_gt + before_gt + __popc(bg & lm);
    const unsigned my_eq = s_base_eq + before_eq + __popc(be & lm);
    // position in the output = (taken above-threshold keys before me) + (taken equal keys before me)
    const unsigned eq_taken_before = my_eq < need_eq ? my_eq : need_eq;
    if (gt) out[my_gt + eq_taken_before] = i;
    if (eq && my_eq < need_eq) out[my_gt + my_eq] = i;
    __syncthreads();
    if (tid == 0) {
      s_base_gt += tot_gt;
      s_base_eq += tot_eq;
    }
    __syncthreads();
  }
  if (tid == 0) a.topk_count[t] = a.k;
}

cudaError_t launch_topk(const B200TopkArgs& a, cudaStream_t s) {
  topk_kernel<<<a.rows, 1024, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace b200mono
