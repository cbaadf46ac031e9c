// What an attention layer does to a token's q | k | v row before the attention itself, for
// layers that norm q and k over the WHOLE projection (all heads at once) and may mix their values
// with another layer's:
//
//   q <- q / rms(q) * w_q     over all heads' channels together (w_q [heads * D]); k likewise
//   rotation of the first `rot` channels of every head, pairs (i, i + rot/2), by p * f_i
//       (p the token's position as a float, f fp32 [rot / 2], sine and cosine of the fp32 product)
//   v <- (1 - lambda) v + lambda v_first    (v_first: the same token's row of another layer)
//   q is written in place, k and v go to the token's cache slot (planes of their own widths).
//
// One block a token; sums of squares, the division, angles and the mix are fp32 arithmetic.  Two
// kernels: a channel a thread, and four channels an access where the sizes allow it.
#include "common.cuh"

namespace gf {

struct WideDims {
  int nh, nkv, D, Vd;
  int k_off, v_off;      // columns of a row where k and v start (q starts at 0)
  int rot;               // rotated channels of a head (even; 0: none)
};

template <typename T>
__global__ void qk_wide_prepare_kernel(T* __restrict__ qkv, int ld, WideDims dm,
                                       const float* __restrict__ qw, const float* __restrict__ kw,
                                       float eps, const float* __restrict__ freqs,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ slot_mapping,
                                       T* __restrict__ kpages, T* __restrict__ vpages,
                                       const T* __restrict__ vfirst, int ld_vf,
                                       const float* __restrict__ lambda) {
  extern __shared__ float tab[];                   // cos [rot/2] | sin [rot/2] | 33 for the sums
  const int t = blockIdx.x;
  const int half = dm.rot / 2;
  float* scratch = tab + 2 * half;
  pdl_trigger();
  pdl_wait();
  T* row = qkv + (size_t)t * ld;
  const int nq = dm.nh * dm.D, nk = dm.nkv * dm.D, nv = dm.nkv * dm.Vd;
  if (half > 0) {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freqs[i], &tab[half + i], &tab[i]);
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (qw != nullptr) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
      const float x = to_f32(row[i]);
      sq = fmaf(x, x, sq);
    }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      const float x = to_f32(row[dm.k_off + i]);
      sk = fmaf(x, x, sk);
    }
    inv_q = 1.f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    inv_k = 1.f / sqrtf(block_sum(sk, scratch) / (float)nk + eps);
  }
  __syncthreads();                                 // the table is there; every sum has been read
  const long long slot = slot_mapping != nullptr ? (long long)slot_mapping[t] : -1;
  // q (in place) and k (to the cache): a thread takes a channel, and its partner with it
  for (int which = 0; which < 2; ++which) {
    if (which == 1 && slot < 0) break;
    const int n = which == 0 ? nq : nk;
    const T* src = which == 0 ? row : row + dm.k_off;
    T* dst = which == 0 ? row : kpages + (size_t)slot * nk;
    const float* w = which == 0 ? qw : kw;
    const float inv = which == 0 ? inv_q : inv_k;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int d = i % dm.D;
      if (d >= half && d < dm.rot) continue;       // the second of a pair: its partner writes it
      float a = to_f32(src[i]) * inv;
      if (w != nullptr) a *= w[i];
      if (d < half) {
        float b = to_f32(src[i + half]) * inv;
        if (w != nullptr) b *= w[i + half];
        const float cs = tab[d], sn = tab[half + d];
        dst[i] = from_f32<T>(a * cs - b * sn);
        dst[i + half] = from_f32<T>(b * cs + a * sn);
      } else {
        dst[i] = from_f32<T>(a);
      }
    }
  }
  if (slot < 0) return;
  const float lam = vfirst != nullptr ? *lambda : 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v = to_f32(row[dm.v_off + i]);
    if (vfirst != nullptr) v = (1.f - lam) * v + lam * to_f32(vfirst[(size_t)t * ld_vf + i]);
    vpages[(size_t)slot * nv + i] = from_f32<T>(v);
  }
}

// The same with four channels an access.  Every run of channels starts on a multiple of four: D,
// Vd, rot / 2, k_off, v_off and the row strides are multiples of four and the pointers aligned to
// four elements.  Work items of the second pass, all in one loop: a quad of a rotated pair's first
// half together with its partner quad, a quad of the channels behind the rotated ones, a quad of
// values.
template <typename T>
__global__ void __launch_bounds__(512)
qk_wide_prepare_vec_kernel(T* __restrict__ qkv, int ld, WideDims dm, const float* __restrict__ qw,
                           const float* __restrict__ kw, float eps,
                           const float* __restrict__ freqs, const int* __restrict__ positions,
                           const int* __restrict__ slot_mapping, T* __restrict__ kpages,
                           T* __restrict__ vpages, const T* __restrict__ vfirst, int ld_vf,
                           const float* __restrict__ lambda) {
  extern __shared__ float tab[];                   // cos [rot/2] | sin [rot/2] | 33 for the sums
  const int t = blockIdx.x;
  const int half = dm.rot / 2;
  float* scratch = tab + 2 * half;
  pdl_trigger();
  pdl_wait();
  T* row = qkv + (size_t)t * ld;
  const int nq = dm.nh * dm.D, nk = dm.nkv * dm.D, nv = dm.nkv * dm.Vd;
  if (half > 0) {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freqs[i], &tab[half + i], &tab[i]);
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (qw != nullptr) {
    float sq = 0.f, sk = 0.f;
    const int qq = nq >> 2, kq = nk >> 2;
    for (int i = threadIdx.x; i < qq + kq; i += blockDim.x) {
      float x[4];
      const bool isk = i >= qq;
      Quad<T>::load(isk ? row + dm.k_off + 4 * (i - qq) : row + 4 * i, x);
      const float s = fmaf(x[0], x[0], fmaf(x[1], x[1], fmaf(x[2], x[2], x[3] * x[3])));
      if (isk) sk += s; else sq += s;
    }
    inv_q = 1.f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    inv_k = 1.f / sqrtf(block_sum(sk, scratch) / (float)nk + eps);
  }
  __syncthreads();                                 // the table is there; every sum has been read
  const long long slot = slot_mapping != nullptr ? (long long)slot_mapping[t] : -1;
  const int hq = half >> 2, ipq = hq + ((dm.D - dm.rot) >> 2);       // items a head
  const int items_q = dm.nh * ipq, items_k = slot >= 0 ? dm.nkv * ipq : 0;
  const int items_v = slot >= 0 ? nv >> 2 : 0;
  const float lam = vfirst != nullptr ? *lambda : 0.f;
  for (int it = threadIdx.x; it < items_q + items_k + items_v; it += blockDim.x) {
    if (it >= items_q + items_k) {                 // values: mixed, to the cache
      const int i = 4 * (it - items_q - items_k);
      float v[4];
      Quad<T>::load(row + dm.v_off + i, v);
      if (vfirst != nullptr) {
        float f[4];
        Quad<T>::load(vfirst + (size_t)t * ld_vf + i, f);
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (1.f - lam) * v[u] + lam * f[u];
      }
      Quad<T>::store(vpages + (size_t)slot * nv + i, v);
      continue;
    }
    const bool isk = it >= items_q;
    const int j = isk ? it - items_q : it;
    const int head = j / ipq, e = j - head * ipq;
    const T* src = isk ? row + dm.k_off : row;
    T* dst = isk ? kpages + (size_t)slot * nk : row;
    const float* w = isk ? kw : qw;
    const float inv = isk ? inv_k : inv_q;
    if (e < hq) {                                  // a rotated quad and its partner
      const int d = 4 * e, i = head * dm.D + d;
      float a[4], b[4];
      Quad<T>::load(src + i, a);
      Quad<T>::load(src + i + half, b);
#pragma unroll
      for (int u = 0; u < 4; ++u) a[u] *= inv, b[u] *= inv;
      if (w != nullptr) {
        float wa[4], wb[4];
        Quad<float>::load(w + i, wa);
        Quad<float>::load(w + i + half, wb);
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] *= wa[u], b[u] *= wb[u];
      }
      float ra[4], rb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float cs = tab[d + u], sn = tab[half + d + u];
        ra[u] = a[u] * cs - b[u] * sn;
        rb[u] = b[u] * cs + a[u] * sn;
      }
      Quad<T>::store(dst + i, ra);
      Quad<T>::store(dst + i + half, rb);
    } else {                                       // behind the rotated channels
      const int i = head * dm.D + dm.rot + 4 * (e - hq);
      float a[4];
      Quad<T>::load(src + i, a);
#pragma unroll
      for (int u = 0; u < 4; ++u) a[u] *= inv;
      if (w != nullptr) {
        float wa[4];
        Quad<float>::load(w + i, wa);
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] *= wa[u];
      }
      Quad<T>::store(dst + i, a);
    }
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// qkv: [T, ld] rows q | .. k at k_off .. v at v_off.  qw / kw: fp32 norm weights or null (no
// norm).  freqs: fp32 [rot / 2] or null.  slot_mapping null: nothing is written to the cache.
// kpages / vpages: [slots, nkv, D] and [slots, nkv, Vd].  vfirst: rows of nkv * Vd values to mix
// in (row stride ld_vf) with the weight *lambda, or null.
GF_EXPORT int gf_qk_wide_prepare(void* qkv, int ld, int T, int nh, int nkv, int D, int Vd,
                                 int k_off, int v_off, const float* qw, const float* kw, float eps,
                                 const float* freqs, int rot, const int* positions,
                                 const int* slot_mapping, void* kpages, void* vpages,
                                 const void* vfirst, int ld_vf, const float* lambda, int dtype,
                                 void* stream) {
  if (T <= 0) return 0;
  if (rot % 2 || rot > D || rot < 0 || (rot > 0 && freqs == nullptr)) return -3;
  WideDims dm;
  dm.nh = nh, dm.nkv = nkv, dm.D = D, dm.Vd = Vd, dm.k_off = k_off, dm.v_off = v_off, dm.rot = rot;
  const size_t smem = (size_t)(rot + 33) * sizeof(float);
  auto st = (cudaStream_t)stream;
  const dim3 grid(T);
  // four channels an access where every run of channels starts on a multiple of four elements
  auto quads = [](const void* p, size_t elem) { return ((uintptr_t)p % (4 * elem)) == 0; };
  const size_t es = dtype == GF_F32 ? 4 : 2;
  const bool vec = D % 4 == 0 && Vd % 4 == 0 && rot % 8 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                   ld % 4 == 0 && quads(qkv, es) && quads(kpages, es) && quads(vpages, es) &&
                   (vfirst == nullptr || (ld_vf % 4 == 0 && quads(vfirst, es))) &&
                   quads(qw, 4) && quads(kw, 4);
  if (vec) {
    const int items = (nh + nkv) * ((rot / 2 + D - rot) / 4) + nkv * Vd / 4;
    const dim3 vblock(items > 256 ? 512 : (items > 128 ? 256 : 128));
    if (dtype == GF_F32)
      return launch_kernel(qk_wide_prepare_vec_kernel<float>, grid, vblock, smem, st, (float*)qkv,
                           ld, dm, qw, kw, eps, freqs, positions, slot_mapping, (float*)kpages,
                           (float*)vpages, (const float*)vfirst, ld_vf, lambda);
    return launch_kernel(qk_wide_prepare_vec_kernel<__nv_bfloat16>, grid, vblock, smem, st,
                         (__nv_bfloat16*)qkv, ld, dm, qw, kw, eps, freqs, positions, slot_mapping,
                         (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages,
                         (const __nv_bfloat16*)vfirst, ld_vf, lambda);
  }
  const dim3 block(256);
  if (dtype == GF_F32)
    return launch_kernel(qk_wide_prepare_kernel<float>, grid, block, smem, st, (float*)qkv, ld, dm,
                         qw, kw, eps, freqs, positions, slot_mapping, (float*)kpages,
                         (float*)vpages, (const float*)vfirst, ld_vf, lambda);
  return launch_kernel(qk_wide_prepare_kernel<__nv_bfloat16>, grid, block, smem, st,
                       (__nv_bfloat16*)qkv, ld, dm, qw, kw, eps, freqs, positions, slot_mapping,
                       (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages,
                       (const __nv_bfloat16*)vfirst, ld_vf, lambda);
}
