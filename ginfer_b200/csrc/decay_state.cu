// Linear recurrences with decays over per-request state, for packed tokens of several requests:
//
//     S_t = diag(g_t) S_(t-1) + (c_t k_t) v_t^T        S: [D, Vd] a head, fp32, in the request's slot
//     o_t = S_t^T q_t + skip_h v_t
//
// g_t is one decay per key channel (gated linear attention) or one per head (state-space duality:
// k = B_t, q = C_t, c = the step size, skip = D_h).  q and k may be shared by groups of heads.
//
//   ssd_prepare_kernel        a thread a (token, channel): causal convolution over time (taps from
//                             this step's rows, or from the slot where the portion starts later than
//                             the tap reaches) + bias + SiLU on the x | B | C channels; step size
//                             dt = softplus(dt + dt_bias) and decay exp(-exp(A_log_h) dt) per head.
//   conv_state_kernel         a thread a (request, channel): the slot's last inputs after the step.
//   gla_prepare_kernel        q * D^-1/2, k, v as fp32 and the decays sigmoid(z)^(1/tau) =
//                             exp(log_sigmoid(z) / tau).
//   decay_recurrence_kernel   a block a (request, head, tile of columns), token after token.  The
//                             columns of S are independent: LP lanes share a column (DPER
//                             neighbouring rows each, in registers) and add their shares of o up by
//                             shuffles, four tokens' shares at a time, off the chain the next token
//                             waits for; the tokens' operands come a chunk ahead through two stages
//                             of shared memory (cp.async, 16 bytes a copy where rows are aligned)
//                             and leave it four floats a load.  Lanes of a warp are laid out
//                             [LP][32 / LP columns], so that a row of S is read and written in
//                             whole 32-byte sectors (LP = 4).
//   gated_norm_kernel         a warp a (token, group of channels): RMS norm with a gate, the gate
//                             before the norm (y = o silu(z), then y / rms(y) w) or behind it
//                             (o / rms(o) w silu(z)); the weight per channel or shared by the groups.
//   gated_norm_block_kernel   the same with a block a (token, group), for groups over 512 channels;
//   gated_norm_vec_kernel     with four channels an access and up to 1,024 threads where rows allow.
//
// Everything here is fp32 arithmetic in both paths; only the projections that feed it and the
// result of gated_norm_kernel have the activation dtype.
#include "common.cuh"

namespace gf {

using bf = __nv_bfloat16;

__device__ __forceinline__ float ds_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float ds_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
// The gate of a gated norm: z * sigmoid(z) (SiLU), or sigmoid(z) alone.
__device__ __forceinline__ float ds_gate(float z, int sigmoid_only) {
  const float sg = ds_sigmoid(z);
  return sigmoid_only ? sg : z * sg;
}
__device__ __forceinline__ float ds_log_sigmoid(float x) {
  return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

struct SsdDims {
  int H, taps;
  int channels;          // convolved columns (x | B | C) of a projection row
  int conv_col;          // where they start in a projection row
  int dt_col;            // where the H step sizes start
  int state_stride;      // floats a slot
  int conv_off;          // where the convolution inputs start in a slot
};

template <typename T>
__global__ void ssd_prepare_kernel(const T* __restrict__ proj, int ld,
                                   const float* __restrict__ conv_w,
                                   const float* __restrict__ conv_b,
                                   const float* __restrict__ dt_bias,
                                   const float* __restrict__ A_log,
                                   const float* __restrict__ state,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ slot_ids, SsdDims dm,
                                   float* __restrict__ xbc, float* __restrict__ rates) {
  const int r = blockIdx.x;
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const int CH = dm.channels, H = dm.H, taps = dm.taps;
  if (ch >= CH + H) return;
  if (ch >= CH) {                                  // a head's step size and decay
    const int h = ch - CH;
    const float dt = ds_softplus(to_f32(proj[(size_t)r * ld + dm.dt_col + h]) + dt_bias[h]);
    rates[(size_t)r * 2 * H + h] = expf(-expf(A_log[h]) * dt);
    rates[(size_t)r * 2 * H + H + h] = dt;
    return;
  }
  const int b = seq_of_token[r];
  const int i = r - cu_seqlens[b];                 // place in this step's portion
  const float* cs = state + (size_t)slot_ids[b] * dm.state_stride + dm.conv_off;
  float acc = conv_b[ch];
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;
    const int off = i - back;                      // place of the tap's input in the portion
    const float x = off >= 0 ? to_f32(proj[(size_t)(r - back) * ld + dm.conv_col + ch])
                             : cs[(size_t)(taps - 1 + off) * CH + ch];
    acc = fmaf(conv_w[(size_t)ch * taps + j], x, acc);
  }
  xbc[(size_t)r * CH + ch] = acc * ds_sigmoid(acc);
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state,
                                  const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ slot_ids, SsdDims dm) {
  const int b = blockIdx.y;
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_trigger();
  pdl_wait();
  if (ch >= dm.channels) return;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  float* cs = state + (size_t)slot_ids[b] * dm.state_stride + dm.conv_off;
  const int keep = dm.taps - 1;
  // entry m holds the input (keep - m) tokens before the next one; ascending m reads only
  // entries that are not yet overwritten
  for (int m = 0; m < keep; ++m) {
    const int idx = n - keep + m;                  // place in the portion, or before it
    cs[(size_t)m * dm.channels + ch] =
        idx >= 0 ? to_f32(proj[(size_t)(start + idx) * ld + dm.conv_col + ch])
                 : cs[(size_t)(m + n) * dm.channels + ch];
  }
}

// proj: q [H D] | k [H D] | v [H Vd] first in a row; z [T, H D] fp32.  out: [T, 3 H D + H Vd] fp32
// laid out q | k | g | v.
template <typename T>
__global__ void gla_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ z,
                                   int rows, int HD, int HV, float q_scale, float inv_tau,
                                   float* __restrict__ out) {
  const int width = 3 * HD + HV;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_trigger();
  pdl_wait();
  if (i >= (size_t)rows * width) return;
  const int r = (int)(i / width), c = (int)(i - (size_t)r * width);
  float y;
  if (c < HD) y = to_f32(proj[(size_t)r * ld + c]) * q_scale;
  else if (c < 2 * HD) y = to_f32(proj[(size_t)r * ld + c]);
  else if (c < 3 * HD) y = expf(ds_log_sigmoid(z[(size_t)r * HD + c - 2 * HD]) * inv_tau);
  else y = to_f32(proj[(size_t)r * ld + c - HD]);
  out[i] = y;
}

// out[r, c] = silu(proj[r, c]) in fp32 for the first `width` columns of a projection row: the q, k
// and v of a linear attention whose operands pass an activation and no other preparation.
template <typename T>
__global__ void silu_f32_kernel(const T* __restrict__ proj, int ld, int rows, int width,
                                float* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_trigger();
  pdl_wait();
  if (i >= (size_t)rows * width) return;
  const int r = (int)(i / width), c = (int)(i - (size_t)r * width);
  const float z = to_f32(proj[(size_t)r * ld + c]);
  out[i] = z * ds_sigmoid(z);
}

// The same from bfloat16 rows, eight channels a thread (one 16-byte load, two 16-byte stores):
// width and ld multiples of 8, aligned rows.
__global__ void silu_f32_vec_kernel(const __nv_bfloat16* __restrict__ proj, int ld, int rows,
                                    int width, float* __restrict__ out) {
  const int w8 = width >> 3;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // No early trigger: the recurrence that follows is a few long-lived blocks, each a chain of
  // dependent steps.  Let in while this grid still fills the SMs, they land several to an SM on
  // the first SMs that drain and the chains share issue slots (measured on a 2,048-token prompt:
  // the recurrence then takes twice as long); after this grid's end they spread one to an SM.
  pdl_wait();
  if (i >= (size_t)rows * w8) return;
  const int r = (int)(i / w8), c = (int)(i - (size_t)r * w8) * 8;
  const uint4 raw = *reinterpret_cast<const uint4*>(proj + (size_t)r * ld + c);
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float z[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    z[2 * j] = f.x * ds_sigmoid(f.x);
    z[2 * j + 1] = f.y * ds_sigmoid(f.y);
  }
  float4* dst = reinterpret_cast<float4*>(out + (size_t)r * width + c);
  dst[0] = make_float4(z[0], z[1], z[2], z[3]);
  dst[1] = make_float4(z[4], z[5], z[6], z[7]);
}

// ------------------------------------------------------------------------------- the recurrence
struct DecayDims {
  int H, G, D, Vd;
  int gD;                // D: a decay a key channel; 1: a decay a head
  int ld_q, ld_k, ld_v, ld_g, ld_c;   // floats between the rows of two tokens
  int state_stride;
};

__device__ __forceinline__ void ds_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void ds_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void ds_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ds_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

constexpr int kDecayWarps = 4;
constexpr int kDecayChunk = 8;
constexpr int kGatedNormWarpMax = 512;           // channels a group one warp still norms
constexpr int kDecayUnroll = 4;                    // tokens whose read-outs are reduced together

// A lane owns the DPER neighbouring rows lp * DPER .. of its column, so that the tokens' q, k and
// decays come out of shared memory four at a time.  VEC: every operand row starts on a 16-byte
// boundary and sizes are multiples of four, so the stages are filled by 16-byte copies.
template <int DPER, int LP, bool VEC>
__global__ void __launch_bounds__(kDecayWarps * 32)
decay_recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k,
                        const float* __restrict__ v, const float* __restrict__ g,
                        const float* __restrict__ c, const float* __restrict__ skip,
                        float* __restrict__ state, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ slot_ids, DecayDims dm, float* __restrict__ o,
                        int ld_o) {
  constexpr int CW = 32 / LP;                      // columns a warp
  constexpr int VT = kDecayWarps * CW;             // columns a block
  constexpr int DP = DPER * LP;                    // key channels, padded
  constexpr int ROW = 3 * DP + VT + 4;             // floats a token in a stage: q | k | g | v | c
  constexpr int P = VEC ? 4 : 1;                   // floats a copy
  extern __shared__ __align__(16) float stage[];   // [2][kDecayChunk][ROW]
  const int b = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lp = lane / CW, vc = lane - lp * CW;
  const int col0 = blockIdx.x * VT;
  const int col = col0 + warp * CW + vc;
  const int D = dm.D, Vd = dm.Vd, gk = h / (dm.H / dm.G);
  const bool live = col < Vd, perch = dm.gD != 1;
  // what cp.async never writes stays zero for ever: the padding rows of q, k and the decays, and
  // the columns past the last one
  for (int i = threadIdx.x; i < 2 * kDecayChunk * ROW; i += blockDim.x) {
    const int e = i % ROW;
    if (e >= 3 * DP || (e % DP) >= D) stage[i] = 0.f;
  }
  pdl_trigger();
  pdl_wait();
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  float* S = state + (size_t)slot_ids[b] * dm.state_stride + (size_t)h * D * Vd;
  float s[DPER];
#pragma unroll
  for (int i = 0; i < DPER; ++i) {
    const int d = lp * DPER + i;
    s[i] = (live && d < D) ? S[(size_t)d * Vd + col] : 0.f;
  }
  const float sk = skip != nullptr ? skip[h] : 0.f;
  __syncthreads();

  auto copy = [&](float* dst, const float* src) {
    if constexpr (VEC) ds_copy16(dst, src); else ds_copy4(dst, src);
  };
  const int dq = D / P, gq = perch ? dq : 0, per = 2 * dq + gq + VT / P;
  auto fetch = [&](int chunk, int buf) {           // a warp a token, a lane a piece
    const int t0 = chunk * kDecayChunk;
    const int cnt = min(kDecayChunk, n - t0);
    float* base = stage + (size_t)buf * kDecayChunk * ROW;
    for (int t = warp; t < cnt; t += kDecayWarps) {
      const size_t r = (size_t)(start + t0 + t);
      float* row = base + t * ROW;
      for (int e = lane; e < per; e += 32) {
        if (e < dq) copy(row + e * P, q + r * dm.ld_q + (size_t)gk * D + e * P);
        else if (e < 2 * dq)
          copy(row + DP + (e - dq) * P, k + r * dm.ld_k + (size_t)gk * D + (e - dq) * P);
        else if (e < 2 * dq + gq)
          copy(row + 2 * DP + (e - 2 * dq) * P, g + r * dm.ld_g + (size_t)h * D + (e - 2 * dq) * P);
        else {
          const int cc = (e - 2 * dq - gq) * P;
          if (col0 + cc < Vd) copy(row + 3 * DP + cc, v + r * dm.ld_v + (size_t)h * Vd + col0 + cc);
        }
      }
      if (lane == 0 && !perch) ds_copy4(row + 2 * DP, g + r * dm.ld_g + h);
      if (lane == 1 && c != nullptr) ds_copy4(row + 3 * DP + VT, c + r * dm.ld_c + h);
    }
    ds_commit();
  };

  // one token: the state's rows of this lane move on, and the lane's share of the read-out
  auto advance = [&](const float* row, float& vv) -> float {
    vv = row[3 * DP + warp * CW + vc];
    const float kv = (c != nullptr ? row[3 * DP + VT] : 1.f) * vv;
    const float g1 = row[2 * DP];
    const float* qr = row + lp * DPER;
    float acc = 0.f;
    if constexpr (DPER % 4 == 0) {
#pragma unroll
      for (int i = 0; i < DPER; i += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
        const float4 k4 = *reinterpret_cast<const float4*>(qr + DP + i);
        const float4 g4 = perch ? *reinterpret_cast<const float4*>(qr + 2 * DP + i)
                                : make_float4(g1, g1, g1, g1);
        s[i] = fmaf(g4.x, s[i], k4.x * kv);
        s[i + 1] = fmaf(g4.y, s[i + 1], k4.y * kv);
        s[i + 2] = fmaf(g4.z, s[i + 2], k4.z * kv);
        s[i + 3] = fmaf(g4.w, s[i + 3], k4.w * kv);
        acc = fmaf(s[i], q4.x, acc);
        acc = fmaf(s[i + 1], q4.y, acc);
        acc = fmaf(s[i + 2], q4.z, acc);
        acc = fmaf(s[i + 3], q4.w, acc);
      }
    } else {
#pragma unroll
      for (int i = 0; i < DPER; ++i) {
        const float gd = perch ? qr[2 * DP + i] : g1;
        s[i] = fmaf(gd, s[i], qr[DP + i] * kv);
        acc = fmaf(s[i], qr[i], acc);
      }
    }
    return acc;
  };

  const int chunks = (n + kDecayChunk - 1) / kDecayChunk;
  if (chunks > 0) fetch(0, 0);
  for (int ch = 0; ch < chunks; ++ch) {
    ds_wait_all();
    __syncthreads();                               // chunk ch has landed; the other stage is free
    if (ch + 1 < chunks) fetch(ch + 1, (ch + 1) & 1);
    const float* base = stage + (size_t)(ch & 1) * kDecayChunk * ROW;
    const int cnt = min(kDecayChunk, n - ch * kDecayChunk);
    float* orow = o + (size_t)(start + ch * kDecayChunk) * ld_o + (size_t)h * Vd + col;
    int t = 0;
    for (; t + kDecayUnroll <= cnt; t += kDecayUnroll) {
      float acc[kDecayUnroll], vv[kDecayUnroll];
#pragma unroll
      for (int u = 0; u < kDecayUnroll; ++u) acc[u] = advance(base + (t + u) * ROW, vv[u]);
#pragma unroll
      for (int off = CW; off < 32; off <<= 1)
#pragma unroll
        for (int u = 0; u < kDecayUnroll; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], off);
      if (lp == 0 && live)
#pragma unroll
        for (int u = 0; u < kDecayUnroll; ++u)
          orow[(size_t)(t + u) * ld_o] = fmaf(sk, vv[u], acc[u]);
    }
    for (; t < cnt; ++t) {
      float vv;
      float acc = advance(base + t * ROW, vv);
#pragma unroll
      for (int off = CW; off < 32; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (lp == 0 && live) orow[(size_t)t * ld_o] = fmaf(sk, vv, acc);
    }
  }
#pragma unroll
  for (int i = 0; i < DPER; ++i) {
    const int d = lp * DPER + i;
    if (live && d < D) S[(size_t)d * Vd + col] = s[i];
  }
}

// ------------------------------------------------------------------------------- gated norm
// o [rows, C] fp32; gate [rows, ...] (G = float or bf16) with row stride gate_ld; groups of gs
// channels; w [C] or, shared, [gs].
template <typename G, typename T>
__global__ void gated_norm_kernel(const float* __restrict__ o, const G* __restrict__ gate,
                                  int gate_ld, const float* __restrict__ w, int w_shared,
                                  int gate_mode, float eps, T* __restrict__ out, int units,
                                  int groups, int gs) {
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int sig = gate_mode >> 1, gate_first = gate_mode & 1;
  pdl_trigger();
  pdl_wait();
  if (unit >= units) return;
  const int r = unit / groups, gi = unit - r * groups;
  const float* orow = o + (size_t)r * groups * gs + (size_t)gi * gs;
  const G* grow = gate + (size_t)r * gate_ld + (size_t)gi * gs;
  T* dst = out + (size_t)r * groups * gs + (size_t)gi * gs;
  float ss = 0.f;
  for (int j = lane; j < gs; j += 32) {
    float y = orow[j];
    if (gate_first) {
      const float z = to_f32(grow[j]);
      y *= ds_gate(z, sig);
    }
    ss = fmaf(y, y, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  for (int j = lane; j < gs; j += 32) {
    const float z = to_f32(grow[j]);
    const float gz = ds_gate(z, sig);
    const float wj = w[w_shared ? j : gi * gs + j];
    const float y = gate_first ? orow[j] * gz * inv * wj : orow[j] * inv * wj * gz;
    dst[j] = from_f32<T>(y);
  }
}


// The same with a block a unit, for groups of thousands of channels (a warp would walk them alone).
template <typename G, typename T>
__global__ void __launch_bounds__(256)
gated_norm_block_kernel(const float* __restrict__ o, const G* __restrict__ gate, int gate_ld,
                        const float* __restrict__ w, int w_shared, int gate_mode, float eps,
                        T* __restrict__ out, int groups, int gs) {
  __shared__ float scratch[33];
  const int unit = blockIdx.x;
  const int sig = gate_mode >> 1, gate_first = gate_mode & 1;
  pdl_trigger();
  pdl_wait();
  const int r = unit / groups, gi = unit - r * groups;
  const float* orow = o + (size_t)r * groups * gs + (size_t)gi * gs;
  const G* grow = gate + (size_t)r * gate_ld + (size_t)gi * gs;
  T* dst = out + (size_t)r * groups * gs + (size_t)gi * gs;
  float ss = 0.f;
  for (int j = threadIdx.x; j < gs; j += blockDim.x) {
    float y = orow[j];
    if (gate_first) {
      const float z = to_f32(grow[j]);
      y *= ds_gate(z, sig);
    }
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  for (int j = threadIdx.x; j < gs; j += blockDim.x) {
    const float z = to_f32(grow[j]);
    const float gz = ds_gate(z, sig);
    const float wj = w[w_shared ? j : gi * gs + j];
    const float y = gate_first ? orow[j] * gz * inv * wj : orow[j] * inv * wj * gz;
    dst[j] = from_f32<T>(y);
  }
}

// The same with four channels an access and up to 1,024 threads a unit: a thread of a group of
// 4,096 channels waits for one load a pass instead of sixteen in a row.  gs and gate_ld are
// multiples of four and the pointers aligned to four elements.
template <typename G, typename T>
__global__ void __launch_bounds__(1024)
gated_norm_vec_kernel(const float* __restrict__ o, const G* __restrict__ gate, int gate_ld,
                      const float* __restrict__ w, int w_shared, int gate_mode, float eps,
                      T* __restrict__ out, int groups, int gs) {
  __shared__ float scratch[33];
  const int unit = blockIdx.x, nq = gs >> 2;
  const int sig = gate_mode >> 1, gate_first = gate_mode & 1;
  pdl_trigger();
  pdl_wait();
  const int r = unit / groups, gi = unit - r * groups;
  const float* orow = o + (size_t)r * groups * gs + (size_t)gi * gs;
  const G* grow = gate + (size_t)r * gate_ld + (size_t)gi * gs;
  const float* wrow = w + (w_shared ? 0 : (size_t)gi * gs);
  T* dst = out + (size_t)r * groups * gs + (size_t)gi * gs;
  float ss = 0.f;
  for (int q = threadIdx.x; q < nq; q += blockDim.x) {
    float y[4];
    Quad<float>::load(orow + 4 * q, y);
    if (gate_first) {
      float z[4];
      Quad<G>::load(grow + 4 * q, z);
#pragma unroll
      for (int u = 0; u < 4; ++u) y[u] *= ds_gate(z[u], sig);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) ss = fmaf(y[u], y[u], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  for (int q = threadIdx.x; q < nq; q += blockDim.x) {
    float y[4], z[4], wq[4];
    Quad<float>::load(orow + 4 * q, y);
    Quad<G>::load(grow + 4 * q, z);
    Quad<float>::load(wrow + 4 * q, wq);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float gz = ds_gate(z[u], sig);
      y[u] = gate_first ? y[u] * gz * inv * wq[u] : y[u] * inv * wq[u] * gz;
    }
    Quad<T>::store(dst + 4 * q, y);
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// proj: [T, ld]; the convolved channels start at conv_col, the H step sizes at dt_col.  xbc:
// [T, channels] fp32; rates: [T, 2 H] fp32, decays first, then step sizes.  The slots' last inputs
// are brought up to date by a second kernel.
GF_EXPORT int gf_ssd_prepare(const void* proj, int ld, int conv_col, int dt_col,
                             const float* conv_w, const float* conv_b, const float* dt_bias,
                             const float* A_log, float* state, const int* seq_of_token,
                             const int* cu_seqlens, const int* slot_ids, int T, int B, int H,
                             int channels, int taps, int state_stride, int conv_off, float* xbc,
                             float* rates, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (taps < 1) return -3;
  SsdDims dm;
  dm.H = H, dm.taps = taps, dm.channels = channels, dm.conv_col = conv_col, dm.dt_col = dt_col;
  dm.state_stride = state_stride, dm.conv_off = conv_off;
  auto st = (cudaStream_t)stream;
  const dim3 pgrid(T, (channels + H + 255) / 256), pblock(256);
  int rc;
  if (dtype == GF_F32)
    rc = launch_kernel(ssd_prepare_kernel<float>, pgrid, pblock, 0, st, (const float*)proj, ld,
                       conv_w, conv_b, dt_bias, A_log, (const float*)state, seq_of_token,
                       cu_seqlens, slot_ids, dm, xbc, rates);
  else
    rc = launch_kernel(ssd_prepare_kernel<bf>, pgrid, pblock, 0, st, (const bf*)proj, ld, conv_w,
                       conv_b, dt_bias, A_log, (const float*)state, seq_of_token, cu_seqlens,
                       slot_ids, dm, xbc, rates);
  if (rc || taps == 1) return rc;
  const dim3 grid((channels + 127) / 128, B);
  if (dtype == GF_F32)
    return launch_kernel(conv_state_kernel<float>, grid, dim3(128), 0, st, (const float*)proj, ld,
                         state, cu_seqlens, slot_ids, dm);
  return launch_kernel(conv_state_kernel<bf>, grid, dim3(128), 0, st, (const bf*)proj, ld, state,
                       cu_seqlens, slot_ids, dm);
}

GF_EXPORT int gf_gla_prepare(const void* proj, int ld, const float* z, int T, int HD, int HV,
                             float q_scale, float inv_tau, float* out, int dtype, void* stream) {
  if (T <= 0) return 0;
  const size_t total = (size_t)T * (3 * HD + HV);
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(gla_prepare_kernel<float>, grid, block, 0, st, (const float*)proj, ld, z,
                         T, HD, HV, q_scale, inv_tau, out);
  return launch_kernel(gla_prepare_kernel<bf>, grid, block, 0, st, (const bf*)proj, ld, z, T, HD,
                       HV, q_scale, inv_tau, out);
}

GF_EXPORT int gf_silu_f32(const void* proj, int ld, int T, int width, float* out, int dtype,
                          void* stream) {
  if (T <= 0 || width <= 0) return 0;
  const size_t total = (size_t)T * width;
  const dim3 grid((unsigned)((total + 255) / 256)), block(256);
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(silu_f32_kernel<float>, grid, block, 0, st, (const float*)proj, ld, T,
                         width, out);
  if (width % 8 == 0 && ld % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const dim3 vgrid((unsigned)((total / 8 + 255) / 256));
    return launch_kernel(silu_f32_vec_kernel, vgrid, block, 0, st, (const bf*)proj, ld, T, width,
                         out);
  }
  return launch_kernel(silu_f32_kernel<bf>, grid, block, 0, st, (const bf*)proj, ld, T, width, out);
}

// q, k: rows of G heads of D; v: rows of H heads of Vd; g: rows of H x gD decays (gD = D or 1);
// c: rows of H factors on k, or null; skip: H weights of v in the output, or null; state: the
// slots, S [H, D, Vd] first in each.  wide: sixteen lanes a column instead of four (few requests
// with long portions).  Returns -3 for key sizes over 256.
GF_EXPORT int gf_decay_recurrence(const float* q, int ld_q, const float* k, int ld_k,
                                  const float* v, int ld_v, const float* g, int ld_g, int gD,
                                  const float* c, int ld_c, const float* skip, float* state,
                                  int state_stride, const int* cu_seqlens, const int* slot_ids,
                                  int B, int H, int G, int D, int Vd, float* o, int ld_o, int wide,
                                  void* stream) {
  if (B <= 0) return 0;
  if (G <= 0 || H % G || (gD != 1 && gD != D) || D <= 0 || D > 256) return -3;
  DecayDims dm;
  dm.H = H, dm.G = G, dm.D = D, dm.Vd = Vd, dm.gD = gD;
  dm.ld_q = ld_q, dm.ld_k = ld_k, dm.ld_v = ld_v, dm.ld_g = ld_g, dm.ld_c = ld_c;
  dm.state_stride = state_stride;
  auto st = (cudaStream_t)stream;
  const int lp = wide ? 16 : 4;
  const int vt = kDecayWarps * (32 / lp);
  const dim3 grid((Vd + vt - 1) / vt, H, B), block(kDecayWarps * 32);
  auto aligned = [](const float* p, int ld) { return ((uintptr_t)p & 15) == 0 && ld % 4 == 0; };
  const bool vec = D % 4 == 0 && Vd % 4 == 0 && aligned(q, ld_q) && aligned(k, ld_k) &&
                   aligned(v, ld_v) && (gD == 1 || aligned(g, ld_g));
#define GF_GO_V(DPER, LP, VEC)                                                                     \
  {                                                                                                \
    const size_t smem = (size_t)2 * kDecayChunk * (3 * LP * DPER + kDecayWarps * (32 / LP) + 4) *  \
                        sizeof(float);                                                             \
    static OncePerDevice once;                                                                     \
    const int rc = once.run([&] {                                                                  \
      return cudaFuncSetAttribute(decay_recurrence_kernel<DPER, LP, VEC>,                          \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    });                                                                                            \
    if (rc) return rc;                                                                             \
    return launch_kernel(decay_recurrence_kernel<DPER, LP, VEC>, grid, block, smem, st, q, k, v,   \
                         g, c, skip, state, cu_seqlens, slot_ids, dm, o, ld_o);                    \
  }
#define GF_GO(DPER, LP)                                                                            \
  if (lp == LP && D <= LP * DPER) {                                                                \
    if (vec) GF_GO_V(DPER, LP, true)                                                               \
    GF_GO_V(DPER, LP, false)                                                                       \
  }
  GF_GO(4, 4)
  GF_GO(8, 4)
  GF_GO(16, 4)
  GF_GO(32, 4)
  GF_GO(64, 4)
  GF_GO(1, 16)
  GF_GO(2, 16)
  GF_GO(4, 16)
  GF_GO(8, 16)
  GF_GO(16, 16)
#undef GF_GO_V
#undef GF_GO
  return -3;
}

// o: [T, groups * gs] fp32 -> out in the activation dtype.  gate_dtype: the gate's own.
// gate_first: bit 0 = the gate before the norm; bit 1 = the gate is sigmoid(z), not z sigmoid(z).
GF_EXPORT int gf_gated_norm(const float* o, const void* gate, int gate_ld, int gate_dtype,
                            const float* w, int w_shared, int gate_first, float eps, void* out,
                            int T, int groups, int gs, int dtype, void* stream) {
  const int units = T * groups;
  if (units <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const dim3 grid((units + 3) / 4), block(128);
  const bool wide = gs > kGatedNormWarpMax;
  auto quads = [](const void* p, size_t elem) { return ((uintptr_t)p % (4 * elem)) == 0; };
  const bool vec = wide && gs % 4 == 0 && gate_ld % 4 == 0 && quads(o, 4) && quads(w, 4) &&
                   quads(gate, gate_dtype == GF_F32 ? 4 : 2) && quads(out, dtype == GF_F32 ? 4 : 2);
  const int vthreads = gs / 4 >= 1024 ? 1024 : (gs / 4 + 31) / 32 * 32;
#define GF_GO(GT, OT)                                                                              \
  {                                                                                                \
    if (vec)                                                                                       \
      return launch_kernel(gated_norm_vec_kernel<GT, OT>, dim3(units), dim3(vthreads), 0, st, o,   \
                           (const GT*)gate, gate_ld, w, w_shared, gate_first, eps, (OT*)out,       \
                           groups, gs);                                                            \
    if (wide)                                                                                      \
      return launch_kernel(gated_norm_block_kernel<GT, OT>, dim3(units), dim3(256), 0, st, o,      \
                           (const GT*)gate, gate_ld, w, w_shared, gate_first, eps, (OT*)out,       \
                           groups, gs);                                                            \
    return launch_kernel(gated_norm_kernel<GT, OT>, grid, block, 0, st, o, (const GT*)gate,        \
                         gate_ld, w, w_shared, gate_first, eps, (OT*)out, units, groups, gs);      \
  }
  if (gate_dtype == GF_F32 && dtype == GF_F32) GF_GO(float, float)
  if (gate_dtype == GF_F32) GF_GO(float, bf)
  if (dtype == GF_F32) GF_GO(bf, float)
  GF_GO(bf, bf)
#undef GF_GO
}
