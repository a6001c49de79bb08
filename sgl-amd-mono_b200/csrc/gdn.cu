// Gated delta network core of the hybrid layers, for decode (one token per request, state committed in place) and
// verify (a chain of T draft tokens per request, window and state snapshotted after every token, committed
// recurrent state untouched).
//
// conv_chain_kernel: one thread per (request, channel): 4-tap causal convolution over [window(3) | new tokens],
//   SiLU, bf16 out; the window advances in registers.  Verify rounds every tap product to bf16, decode keeps f32.
// delta_chain_kernel: one CTA of 256 threads per (request, value head).  The head's 128x128 f32 state lives in
//   registers for the whole chain: thread (i, half) owns row i and the 16 float4 column chunks 2j+half, so a pair of
//   lanes reads / writes whole 32-byte sectors and a row dot product needs one shuffle.  HBM traffic is the
//   state read once and one snapshot written per token: the roofline of this stage.
#include "common.cuh"
#include "launch.h"

namespace b200mono {

constexpr int kD = 128;

__global__ __launch_bounds__(256) void conv_chain_kernel(B200GdnArgs a) {
  pdl_enter();
  const int req = blockIdx.x;
  const int col = blockIdx.y * 256 + threadIdx.x;
  const int conv_dim = (2 * a.hk + a.hv) * kD;
  if (col >= conv_dim) return;
  const int slot = a.slot[req];
  const int T = a.tokens;
  const __nv_bfloat16* qkvz = reinterpret_cast<const __nv_bfloat16*>(a.qkvz);
  __nv_bfloat16* mixed = reinterpret_cast<__nv_bfloat16*>(a.mixed);
  if (slot < 0) {
    for (int t = 0; t < T; ++t) mixed[(size_t)(req * T + t) * conv_dim + col] = __float2bfloat16_rn(0.f);
    return;
  }
  __nv_bfloat16* cell = reinterpret_cast<__nv_bfloat16*>(a.conv_state) + (size_t)slot * 3 * conv_dim + col;
  float c0 = __bfloat162float(cell[0]), c1 = __bfloat162float(cell[conv_dim]), c2 = __bfloat162float(cell[2 * conv_dim]);
  const uint2 wv = reinterpret_cast<const uint2*>(a.conv_w)[col];
  const float w0 = bf16_lo(wv.x), w1 = bf16_hi(wv.x), w2 = bf16_lo(wv.y), w3 = bf16_hi(wv.y);
  const float bias = a.conv_bias ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.conv_bias)[col]) : 0.f;
  const int islot = a.inter_slot ? a.inter_slot[req] : -1;
  const bool verify = !a.commit;
  for (int t = 0; t < T; ++t) {
    const int row = req * T + t;
    const float x = __bfloat162float(qkvz[(size_t)row * a.qkvz_stride + col]);
    float t0 = __fmul_rn(c0, w0), t1 = __fmul_rn(c1, w1), t2 = __fmul_rn(c2, w2), t3 = __fmul_rn(x, w3);
    if (verify) {
      t0 = round_bf16(t0);
      t1 = round_bf16(t1);
      t2 = round_bf16(t2);
      t3 = round_bf16(t3);
    }
    float acc = __fadd_rn(t0, t1);
    acc = __fadd_rn(__fadd_rn(acc, t2), t3);
    if (a.conv_bias) acc = __fadd_rn(acc, bias);
    const float y = acc / (1.0f + expf(-acc));
    mixed[(size_t)row * conv_dim + col] = __float2bfloat16_rn(y);
    c0 = c1;
    c1 = c2;
    c2 = x;
    if (verify && islot >= 0) {
      __nv_bfloat16* step = reinterpret_cast<__nv_bfloat16*>(a.inter_conv) + ((size_t)islot * T + t) * 3 * conv_dim + col;
      step[0] = __float2bfloat16_rn(c0);
      step[conv_dim] = __float2bfloat16_rn(c1);
      step[2 * conv_dim] = __float2bfloat16_rn(c2);
    }
  }
  cell[0] = __float2bfloat16_rn(c0);
  cell[conv_dim] = __float2bfloat16_rn(c1);
  cell[2 * conv_dim] = __float2bfloat16_rn(c2);
}

// sums N values over the 256 threads of the CTA; every thread gets the totals (warp order 0..7)
template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* buf /* [8*N] */) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int n = 0; n < N; ++n) v[n] = warp_sum_tree(v[n]);
  __syncthreads();  // previous readers of buf are done
  if (lane == 0)
#pragma unroll
    for (int n = 0; n < N; ++n) buf[warp * N + n] = v[n];
  __syncthreads();
#pragma unroll
  for (int n = 0; n < N; ++n) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += buf[w * N + n];
    v[n] = s;
  }
}

__device__ __forceinline__ float block_max(float v, float* buf /* [8] */) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  float m = buf[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, buf[w]);
  return m;
}

constexpr int kMaxTokens = 8;  // tokens of a chain handled per pass (longer chains run in passes)

// Phase A: gate scalars and the normalised q / k of every token of the pass (one round of block sums).
// Phase B: the recurrence, token by token, on the state in registers; snapshots are fire-and-forget stores, so
//          the memory pipe stays busy while the next token's arithmetic runs.
// Phase C: gated RMSNorm + FP8 group of every token (one more round of block sums).
__global__ __launch_bounds__(256, 2) void delta_chain_kernel(B200GdnArgs a) {
  pdl_enter();
  __shared__ __align__(16) float s_q[kMaxTokens][kD], s_k[kMaxTokens][kD], s_v[kMaxTokens][kD], s_o[kMaxTokens][kD];
  __shared__ float s_red[8 * 4 * kMaxTokens];
  __shared__ float s_decay[kMaxTokens], s_beta[kMaxTokens];
  const int req = blockIdx.x, hv = blockIdx.y, tid = threadIdx.x;
  const int i = tid >> 1, half = tid & 1;
  const int HK = a.hk, HV = a.hv, T = a.tokens;
  const int kh = hv / (HV / HK);
  const int conv_dim = (2 * HK + HV) * kD;
  const int slot = a.slot[req];
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
  uint8_t* out_q = reinterpret_cast<uint8_t*>(a.out_q);
  if (slot < 0) {  // dead request: zeros, the scale of an all-zero group
    for (int t = 0; t < T; ++t) {
      const int row = req * T + t;
      if (tid < kD) {
        out[(size_t)row * HV * kD + hv * kD + tid] = __float2bfloat16_rn(0.f);
        out_q[(size_t)row * HV * kD + hv * kD + tid] = 0;
      }
      if (tid == 0) a.out_scale[(size_t)row * HV + hv] = 1e-10f * (1.0f / 448.0f);
    }
    return;
  }
  const bool verify = !a.commit;
  const int islot = (verify && a.inter_slot) ? a.inter_slot[req] : -1;
  float* cell = a.ssm_state + (((size_t)slot * HV + hv) * kD + i) * kD;
  float4 h[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) h[j] = *reinterpret_cast<const float4*>(cell + 4 * (2 * j + half));
  const float a_log = a.a_log[hv], dt_bias = a.dt_bias[hv];
  const float nw = tid < kD ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.norm_w)[tid]) : 0.f;
  const __nv_bfloat16* ba_w = reinterpret_cast<const __nv_bfloat16*>(a.ba_w);
  const __nv_bfloat16* hidden = reinterpret_cast<const __nv_bfloat16*>(a.hidden);
  const __nv_bfloat16* mixed = reinterpret_cast<const __nv_bfloat16*>(a.mixed);
  const __nv_bfloat16* qkvz = reinterpret_cast<const __nv_bfloat16*>(a.qkvz);

  for (int t0 = 0; t0 < T; t0 += kMaxTokens) {
    const int nt = min(kMaxTokens, T - t0);
    // ---- phase A
    float sums[4 * kMaxTokens];
#pragma unroll
    for (int n = 0; n < 4 * kMaxTokens; ++n) sums[n] = 0.f;
    float qv[kMaxTokens], kv[kMaxTokens];
    for (int e = tid * 8; e < a.k_in; e += 256 * 8) {
      const uint4 wb = ld_u4(ba_w + (size_t)hv * a.k_in + e);
      const uint4 wa = ld_u4(ba_w + (size_t)(HV + hv) * a.k_in + e);
      const uint32_t bs[4] = {wb.x, wb.y, wb.z, wb.w}, as[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
      for (int tt = 0; tt < kMaxTokens; ++tt) {
        if (tt < nt) {
          const uint4 xv = ld_u4(hidden + (size_t)(req * T + t0 + tt) * a.k_in + e);
          const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            sums[4 * tt] = fmaf(bf16_lo(xs[p]), bf16_lo(bs[p]), sums[4 * tt]);
            sums[4 * tt] = fmaf(bf16_hi(xs[p]), bf16_hi(bs[p]), sums[4 * tt]);
            sums[4 * tt + 1] = fmaf(bf16_lo(xs[p]), bf16_lo(as[p]), sums[4 * tt + 1]);
            sums[4 * tt + 1] = fmaf(bf16_hi(xs[p]), bf16_hi(as[p]), sums[4 * tt + 1]);
          }
        }
      }
    }
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      qv[tt] = kv[tt] = 0.f;
      if (tt < nt) {
        const size_t row = (size_t)(req * T + t0 + tt);
        if (tid < kD) {
          qv[tt] = __bfloat162float(mixed[row * conv_dim + kh * kD + tid]);
          kv[tt] = __bfloat162float(mixed[row * conv_dim + (HK + kh) * kD + tid]);
          sums[4 * tt + 2] = qv[tt] * qv[tt];
          sums[4 * tt + 3] = kv[tt] * kv[tt];
        } else {
          s_v[tt][tid - kD] = __bfloat162float(mixed[row * conv_dim + (2 * HK) * kD + hv * kD + tid - kD]);
        }
      }
    }
    block_sum<4 * kMaxTokens>(sums, s_red);
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      if (tt < nt) {
        if (tid < kD) {
          s_q[tt][tid] = qv[tt] / sqrtf(sums[4 * tt + 2] + 1e-6f) * a.scale;
          s_k[tt][tid] = kv[tt] / sqrtf(sums[4 * tt + 3] + 1e-6f);
        }
        if (tid == 0) {
          const float bb = round_bf16(sums[4 * tt]), aa = round_bf16(sums[4 * tt + 1]);
          const float x = aa + dt_bias;
          const float softplus = x <= 20.0f ? log1pf(expf(x)) : x;
          s_decay[tt] = expf(-expf(a_log) * softplus);
          const float beta = 1.0f / (1.0f + expf(-bb));
          s_beta[tt] = verify ? beta : round_bf16(beta);
        }
      }
    }
    __syncthreads();
    // ---- phase B:  S <- S * decay;  v' = (v - S k) * beta;  S <- S + v' (x) k;  o = S q
    for (int tt = 0; tt < nt; ++tt) {
      const float decay = s_decay[tt], beta = s_beta[tt];
      float hk_part = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 kk = *reinterpret_cast<const float4*>(&s_k[tt][4 * (2 * j + half)]);
        h[j].x *= decay;
        h[j].y *= decay;
        h[j].z *= decay;
        h[j].w *= decay;
        hk_part = fmaf(h[j].x, kk.x, hk_part);
        hk_part = fmaf(h[j].y, kk.y, hk_part);
        hk_part = fmaf(h[j].z, kk.z, hk_part);
        hk_part = fmaf(h[j].w, kk.w, hk_part);
      }
      const float hk_full = hk_part + __shfl_xor_sync(0xffffffffu, hk_part, 1);
      const float vn = (s_v[tt][i] - hk_full) * beta;
      float o_part = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 kk = *reinterpret_cast<const float4*>(&s_k[tt][4 * (2 * j + half)]);
        const float4 qq = *reinterpret_cast<const float4*>(&s_q[tt][4 * (2 * j + half)]);
        h[j].x = fmaf(vn, kk.x, h[j].x);
        h[j].y = fmaf(vn, kk.y, h[j].y);
        h[j].z = fmaf(vn, kk.z, h[j].z);
        h[j].w = fmaf(vn, kk.w, h[j].w);
        o_part = fmaf(h[j].x, qq.x, o_part);
        o_part = fmaf(h[j].y, qq.y, o_part);
        o_part = fmaf(h[j].z, qq.z, o_part);
        o_part = fmaf(h[j].w, qq.w, o_part);
      }
      const float o_full = o_part + __shfl_xor_sync(0xffffffffu, o_part, 1);
      if (half == 0) s_o[tt][i] = round_bf16(o_full);
      if (islot >= 0) {
        float* snap = a.inter_ssm + ((((size_t)islot * T + t0 + tt) * HV + hv) * kD + i) * kD;
#pragma unroll
        for (int j = 0; j < 16; ++j) __stcs(reinterpret_cast<float4*>(snap + 4 * (2 * j + half)), h[j]);
      }
    }
    __syncthreads();
    // ---- phase C: gated RMSNorm over the head's 128 outputs, then the FP8 group of the next projection
    float ss[kMaxTokens], yf[kMaxTokens];
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      const float o = (tt < nt && tid < kD) ? s_o[tt][tid] : 0.f;
      ss[tt] = o * o;
    }
    block_sum<kMaxTokens>(ss, s_red);
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      yf[tt] = 0.f;
      if (tt < nt && tid < kD) {
        const size_t row = (size_t)(req * T + t0 + tt);
        const float z = __bfloat162float(qkvz[row * a.qkvz_stride + conv_dim + hv * kD + tid]);
        const float rstd = rsqrtf(ss[tt] / kD + a.eps);
        const float y = s_o[tt][tid] * rstd * nw * (z * (1.0f / (1.0f + expf(-z))));
        yf[tt] = round_bf16(y);
        out[row * HV * kD + hv * kD + tid] = __float2bfloat16_rn(y);
      }
    }
    // group maxima of all tokens: warps 0..3 hold the head's 128 values
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      const float m = warp_max(fabsf(yf[tt]));
      if ((tid & 31) == 0) s_red[(tid >> 5) * kMaxTokens + tt] = m;
    }
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < kMaxTokens; ++tt) {
      if (tt < nt) {
        const size_t row = (size_t)(req * T + t0 + tt);
        const float amax = fmaxf(fmaxf(s_red[tt], s_red[kMaxTokens + tt]), fmaxf(s_red[2 * kMaxTokens + tt], s_red[3 * kMaxTokens + tt]));
        const float gs = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
        const float inv = 1.0f / gs;
        // four neighbours pack one 32-bit store
        const float y1 = __shfl_down_sync(0xffffffffu, yf[tt], 1), y2 = __shfl_down_sync(0xffffffffu, yf[tt], 2),
                    y3 = __shfl_down_sync(0xffffffffu, yf[tt], 3);
        if (tid < kD && (tid & 3) == 0) {
          auto q = [&](float y) { return fminf(fmaxf(y * inv, -448.f), 448.f); };
          *reinterpret_cast<uint32_t*>(out_q + row * HV * kD + hv * kD + tid) = f32x4_to_e4m3x4(q(yf[tt]), q(y1), q(y2), q(y3));
        }
        if (tid == 0) a.out_scale[row * HV + hv] = gs;
      }
    }
    __syncthreads();  // shared arrays are rewritten by the next pass
  }
  if (!verify) {
#pragma unroll
    for (int j = 0; j < 16; ++j) *reinterpret_cast<float4*>(cell + 4 * (2 * j + half)) = h[j];
  }
}

cudaError_t launch_gdn(const B200GdnArgs& a, cudaStream_t s) {
  const int conv_dim = (2 * a.hk + a.hv) * kD;
  dim3 g1(a.requests, (conv_dim + 255) / 256);
  launch_pdl(conv_chain_kernel, g1, 256, 0, s, a);
  dim3 g2(a.requests, a.hv);
  launch_pdl(delta_chain_kernel, g2, 256, 0, s, a);
  return cudaGetLastError();
}

}  // namespace b200mono
