// Weight-streaming block-FP8 GEMV core for M <= 32 activation rows (swap-AB).
//
// A warp owns a tile of 16 weight rows (MMA M) and a range of 128-wide k
// blocks; activation rows are the MMA N dimension, 8 per MMA.  Per k block and
// row set a lane issues two 256-bit streaming loads (rows g and g+8, 32 bytes
// at column 32c), so a warp instruction covers 8 rows x 128 contiguous bytes:
// whole lines, each weight byte requested exactly once, nothing staged in
// shared memory.  Four m16n8k32 e4m3 MMAs accumulate the 128-k partial, which
// is then folded into the running sum with the f32 block scale
// ws[n/128][k/128] * xs[t][k/128] (128x128 f32 scales are not an MX format, so
// the scale is applied on the accumulator, once per k block).  Loads of block
// kb+1 are in flight while block kb is multiplied.
#pragma once
#include "common.cuh"

namespace b200mono {

template <int R>
struct WFrag {
  U256 v[R][2];  // [row set][rows g / g+8]
};

// p[r] points at byte (row g of the tile, column 32c) of row set r.
template <int R, bool HALF>
__device__ __forceinline__ void load_wfrag(WFrag<R>& f, const uint8_t* const (&p)[R], size_t ldw,
                                           int kb) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint8_t* q = p[r] + (size_t)kb * 128;
    f.v[r][0] = ld_stream_u256(q);
    if (!HALF) {
      f.v[r][1] = ld_stream_u256(q + 8 * ldw);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f.v[r][1].v[i] = 0;
    }
  }
}

// Activation view of one warp: row t = nt*8 + g feeds MMA column g.
template <int NT>
struct XView {
  const uint8_t* row[NT];  // byte (row nt*8+g, column 32c) or nullptr past the last row
  const float* s0[NT];     // scale row of t = nt*8 + 2c   (nullptr past the last row)
  const float* s1[NT];     // scale row of t = nt*8 + 2c+1
};

template <int NT>
__device__ __forceinline__ XView<NT> make_xview(const uint8_t* x, size_t ldx, const float* xs,
                                                size_t ldxs, int rows, int lane) {
  XView<NT> v;
  const int g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    int t = nt * 8 + g;
    v.row[nt] = t < rows ? x + (size_t)t * ldx + 32 * c : nullptr;
    int t0 = nt * 8 + 2 * c;
    v.s0[nt] = t0 < rows ? xs + (size_t)t0 * ldxs : nullptr;
    v.s1[nt] = t0 + 1 < rows ? xs + (size_t)(t0 + 1) * ldxs : nullptr;
  }
  return v;
}

// One 128-k block: acc[r][nt][i] += (W_tile . x) * ws[r] * xs.
template <int R, int NT>
__device__ __forceinline__ void mma_block(const WFrag<R>& w, const XView<NT>& xv, int kb,
                                          const float (&ws)[R], float (&acc)[R][NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
    if (xv.row[nt]) {
      x0 = ld_u4(xv.row[nt] + (size_t)kb * 128);
      x1 = ld_u4(xv.row[nt] + (size_t)kb * 128 + 16);
    }
    float s0 = xv.s0[nt] ? xv.s0[nt][kb] : 0.f;
    float s1 = xv.s1[nt] ? xv.s1[nt][kb] : 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float p[4] = {0.f, 0.f, 0.f, 0.f};
      const U256 &lo = w.v[r][0], &hi = w.v[r][1];
      mma_e4m3_16x8x32(p, lo.v[0], hi.v[0], lo.v[1], hi.v[1], x0.x, x0.y);
      mma_e4m3_16x8x32(p, lo.v[2], hi.v[2], lo.v[3], hi.v[3], x0.z, x0.w);
      mma_e4m3_16x8x32(p, lo.v[4], hi.v[4], lo.v[5], hi.v[5], x1.x, x1.y);
      mma_e4m3_16x8x32(p, lo.v[6], hi.v[6], lo.v[7], hi.v[7], x1.z, x1.w);
      float f0 = ws[r] * s0, f1 = ws[r] * s1;
      acc[r][nt][0] = fmaf(p[0], f0, acc[r][nt][0]);
      acc[r][nt][1] = fmaf(p[1], f1, acc[r][nt][1]);
      acc[r][nt][2] = fmaf(p[2], f0, acc[r][nt][2]);
      acc[r][nt][3] = fmaf(p[3], f1, acc[r][nt][3]);
    }
  }
}

// Stream k blocks [kb0, kb1) of R row sets, two-deep register pipeline.
// wsc[r] points at the scale row ws[(n/128)][0] of row set r.
template <int R, int NT, bool HALF>
__device__ __forceinline__ void stream_tile(const uint8_t* const (&wp)[R], size_t ldw,
                                            const float* const (&wsc)[R], const XView<NT>& xv,
                                            int kb0, int kb1, float (&acc)[R][NT][4]) {
  if (kb0 >= kb1) return;
  WFrag<R> f0, f1;
  load_wfrag<R, HALF>(f0, wp, ldw, kb0);
  int kb = kb0;
  for (; kb + 1 < kb1; kb += 2) {
    load_wfrag<R, HALF>(f1, wp, ldw, kb + 1);
    float ws[R];
#pragma unroll
    for (int r = 0; r < R; ++r) ws[r] = wsc[r][kb];
    mma_block<R, NT>(f0, xv, kb, ws, acc);
    if (kb + 2 < kb1) load_wfrag<R, HALF>(f0, wp, ldw, kb + 2);
#pragma unroll
    for (int r = 0; r < R; ++r) ws[r] = wsc[r][kb + 1];
    mma_block<R, NT>(f1, xv, kb + 1, ws, acc);
  }
  if (kb < kb1) {
    float ws[R];
#pragma unroll
    for (int r = 0; r < R; ++r) ws[r] = wsc[r][kb];
    mma_block<R, NT>(f0, xv, kb, ws, acc);
  }
}

}  // namespace b200mono
