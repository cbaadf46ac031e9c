// Routed feed-forward (mixture of experts) without a host round trip: every kernel reads the
// routing from device memory, so a step can be captured in a CUDA graph.
//
//   moe_route_kernel    a warp a token: scores = softmax(router logits) in fp32 over all experts
//                       (or the sigmoid of each logit), the `top` largest chosen (lowest index
//                       among equals), their scores kept as weights (optionally renormalised over
//                       the chosen ones).
//   moe_plan_kernel     a block an expert: (token, choice) pairs counted per expert, the experts' ranges in
//                       the sorted order, each pair's place, and the list of row tiles (expert,
//                       first row) that the grouped products walk over.
//   moe_gemm_mma_kernel the grouped products of the bf16 path, on the tensor cores (see there).
//   moe_gemm_kernel     (32-bit path, and sizes the other refuses) grouped product over the sorted pairs, a block a (row tile, column tile):
//                       FIRST: rows gathered from the tokens, W = the expert's row-interleaved
//                       gate/up matrix, epilogue = clamped sigmoid-gated GLU (MODE 1), or W = the
//                       expert's up matrix, epilogue = relu(w * acc)^2 with the pair's routing
//                       weight w, which is the product of the row scaled by w (MODE 2); else
//                       (MODE 0) rows = the first product's output, W = the expert's down matrix,
//                       fp32 out.  The reduction runs in a fixed order, so a pair's result does
//                       not depend on the batch.
//   moe_combine_kernel  out[t] = sum over the token's choices, in the order chosen, of weight *
//                       the pair's row.
#include "common.cuh"

namespace gf {

constexpr int kMaxExperts = 256;
constexpr int kRouteSlots = kMaxExperts / 32;

__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int top,
                                 int renorm, int sigmoid, int* __restrict__ idx,
                                 float* __restrict__ wgt) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (t >= T) return;
  float s[kRouteSlots];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRouteSlots; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
    mx = fmaxf(mx, s[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kRouteSlots; ++i) {
    const float sc = sigmoid ? 1.f / (1.f + expf(-s[i])) : expf(s[i] - mx);
    s[i] = lane + 32 * i < E ? sc : -1.f;                    // -1: no expert, or taken
    sum += s[i] > 0.f ? s[i] : 0.f;
  }
  sum = sigmoid ? 1.f : warp_sum(sum);
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRouteSlots; ++i)
      if (s[i] > best) best = s[i], be = lane + 32 * i;       // ascending e: lowest index wins
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) best = ob, be = oe;
    }
#pragma unroll
    for (int i = 0; i < kRouteSlots; ++i)
      if (lane + 32 * i == be) s[i] = -1.f;
    chosen_sum += best;
    if (lane == 0) {
      idx[(size_t)t * top + k] = be;
      wgt[(size_t)t * top + k] = best / sum;
    }
  }
  if (renorm) {
    __syncwarp();
    if (lane < top) wgt[(size_t)t * top + lane] *= sum / chosen_sum;
  }
}

// Pairs p = t * top + k.  offsets[E + 1]; pos_of_pair[P]; pair_of_pos[P]; tiles: tile_expert[],
// tile_row0[] (first sorted row of the tile), num_tiles[0].
// A block an expert (one SM could not keep up: 8,192 pairs took 29 us in one block).  Every block
// counts all experts' pairs for itself, so that it knows where its expert's rows and tiles begin
// without waiting for another block; then its warps take equal runs of the pairs, count their
// expert's pairs in them, and place them behind the runs before: a pair's place is the number of
// earlier pairs of the same expert, whatever the grid.
constexpr int kPlanThreads = 256, kPlanWarps = kPlanThreads / 32;
__global__ void __launch_bounds__(kPlanThreads)
moe_plan_kernel(const int* __restrict__ idx, int P, int E, int tile_rows,
                int* __restrict__ offsets, int* __restrict__ pos_of_pair,
                int* __restrict__ pair_of_pos, int* __restrict__ tile_expert,
                int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
  __shared__ int count[kMaxExperts], run_count[kPlanWarps], base[2];
  const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  for (int i = threadIdx.x; i < E; i += blockDim.x) count[i] = 0;
  __syncthreads();
  // this block's expert by ballots over the warps' runs; the others by shared atomics
  const int run = (((P + kPlanWarps - 1) / kPlanWarps) + 31) & ~31;
  const int p_lo = warp * run, p_hi = min(P, p_lo + run);
  int mine_in_run = 0;
  for (int p0 = p_lo; p0 < p_hi; p0 += 32) {
    const int p = p0 + lane;
    const int g = p < p_hi ? idx[p] : -1;
    if (g >= 0 && g != e) atomicAdd(&count[g], 1);
    mine_in_run += __popc(__ballot_sync(0xffffffffu, g == e));
  }
  if (lane == 0) run_count[warp] = mine_in_run;
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int w = 0; w < kPlanWarps; ++w) n += run_count[w];
    count[e] = n;
    int at = 0, nt = 0;
    for (int i = 0; i < e; ++i) {
      at += count[i];
      nt += (count[i] + tile_rows - 1) / tile_rows;
    }
    base[0] = at;
    base[1] = nt;
    offsets[e] = at;
    if (e == E - 1) {
      offsets[E] = at + n;
      num_tiles[0] = nt + (n + tile_rows - 1) / tile_rows;
    }
  }
  __syncthreads();
  const int start = base[0], n_mine = count[e];
  for (int r = threadIdx.x * tile_rows; r < n_mine; r += blockDim.x * tile_rows) {
    tile_expert[base[1] + r / tile_rows] = e;
    tile_row0[base[1] + r / tile_rows] = start + r;
  }
  int at = start;
  for (int w = 0; w < warp; ++w) at += run_count[w];
  for (int p0 = p_lo; p0 < p_hi; p0 += 32) {
    const int p = p0 + lane;
    const bool mine = p < p_hi && idx[p] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (mine) {
      const int pos = at + __popc(m & ((1u << lane) - 1));
      pos_of_pair[p] = pos;
      pair_of_pos[pos] = p;
    }
    at += __popc(m);
  }
}

__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha,
                                             float up_shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  if (alpha < 0.f) return fmaxf(g, 0.f) * (u + up_shift);   // the sigmoid sharpened to a step: relu
  return g / (1.f + expf(-alpha * g)) * (u + up_shift);
}

constexpr int kBM = 32, kBN = 64, kBK = 32;

// MODE 1: a [T, K] tokens (row of sorted place s = pair_of_pos[s] / top), w [E, 2F, K] (gate row,
// up row, ...), out [P, F] of type T.  MODE 2: the same rows, w [E, F, K], out [P, F] of type T =
// relu(row_w[pair] * acc)^2 (row_w null: 1).  MODE 0: a [P, K] (T), w [E, N, K], out [P, N] fp32.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ a, int lda, const T* __restrict__ w, int N, int K,
                const int* __restrict__ offsets, const int* __restrict__ pair_of_pos, int top,
                const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                const int* __restrict__ num_tiles, void* __restrict__ out_, float limit,
                float alpha, float up_shift, const float* __restrict__ row_w) {
  constexpr bool FIRST = MODE != 0;
  __shared__ float As[kBM][kBK + 1], Ws[kBN][kBK + 1];
  __shared__ int src_row[kBM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= num_tiles[0]) return;
  const int e = tile_expert[blockIdx.x], row0 = tile_row0[blockIdx.x];
  const int rows = min(kBM, offsets[e + 1] - row0);
  const int n0 = blockIdx.y * kBN;
  const T* we = w + (size_t)e * N * K;
  if (threadIdx.x < kBM) {
    const int s = row0 + threadIdx.x;
    src_row[threadIdx.x] = threadIdx.x < rows ? (FIRST ? pair_of_pos[s] / top : s) : -1;
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;    // rows 2 ty, 2 ty + 1; cols 4 tx ..
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += kBK) {
    for (int i = threadIdx.x; i < kBM * kBK; i += 256) {
      const int r = i / kBK, k = i - r * kBK;
      const int sr = src_row[r];
      As[r][k] = (sr >= 0 && k0 + k < K) ? to_f32(a[(size_t)sr * lda + k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < kBN * kBK; i += 256) {
      const int n = i / kBK, k = i - n * kBK;
      Ws[n][k] = (n0 + n < N && k0 + k < K) ? to_f32(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kBK; ++k) {
      const float a0 = As[2 * ty][k], a1 = As[2 * ty + 1][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Ws[4 * tx + j][k];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = 2 * ty + i;
    if (r >= rows) continue;
    const size_t s = (size_t)(row0 + r);
    if (MODE == 2) {
      T* out = (T*)out_;
      const float rw = row_w ? row_w[pair_of_pos[s]] : 1.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + 4 * tx + j;
        if (n < N) {
          const float u = fmaxf(to_f32(from_f32<T>(acc[i][j] * rw)), 0.f);
          out[s * N + n] = from_f32<T>(u * u);
        }
      }
    } else if (MODE == 1) {
      T* out = (T*)out_;
      const int F = N / 2;
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + 4 * tx + j;
        if (n < N) {
          // gate and up are rounded to the activation type as a plain product would store them
          const float gt = to_f32(from_f32<T>(acc[i][j])), up = to_f32(from_f32<T>(acc[i][j + 1]));
          out[s * F + n / 2] = from_f32<T>(clamped_glu(gt, up, limit, alpha, up_shift));
        }
      }
    } else {
      float* out = (float*)out_;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + 4 * tx + j;
        if (n < N) out[s * N + n] = acc[i][j];
      }
    }
  }
}


// ---- the same grouped products on the tensor cores (bf16 operands, fp32 accumulation) -----------
// Tile 64 rows x 128 columns x 32 of the reduction; 8 warps as 2 x 4, a warp 32 x 32 (2 x 4
// mma.sync.m16n8k16 a k-step).  Operand tiles come through three stages of shared memory by 16-byte
// cp.async (rows 40 halves apart: fragment loads meet every bank once); rows past an expert's range
// are zero-filled.  Needs K and the row strides to be multiples of 8 and 16-byte aligned bases.
constexpr int kTM = 64, kTN = 128, kTK = 32, kTStages = 3, kTLd = kTK + 8;

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n)
               : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                        const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_u32(p)));
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w,
                    int N, int K, const int* __restrict__ offsets,
                    const int* __restrict__ pair_of_pos, int top,
                    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    const int* __restrict__ num_tiles, void* __restrict__ out_, float limit,
                    float alpha, float up_shift, const float* __restrict__ row_w) {
  constexpr bool FIRST = MODE != 0;
  __shared__ __align__(16) __nv_bfloat16 As[kTStages][kTM][kTLd];
  __shared__ __align__(16) __nv_bfloat16 Ws[kTStages][kTN][kTLd];
  __shared__ int src_row[kTM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= num_tiles[0]) return;
  const int e = tile_expert[blockIdx.x], row0 = tile_row0[blockIdx.x];
  const int rows = min(kTM, offsets[e + 1] - row0);
  const int n0 = blockIdx.y * kTN;
  const __nv_bfloat16* we = w + (size_t)e * N * K;
  if (threadIdx.x < kTM) {
    const int s = row0 + threadIdx.x;
    src_row[threadIdx.x] = threadIdx.x < rows ? (FIRST ? pair_of_pos[s] / top : s) : -1;
  }
  __syncthreads();
  const int nk = (K + kTK - 1) / kTK;
  auto ask = [&](int kb) {
    const int st = kb % kTStages, k0 = kb * kTK;
    {                                              // A: 64 rows x 4 pieces of 8
      const int r = threadIdx.x >> 2, c = (threadIdx.x & 3) * 8;
      const int sr = src_row[r];
      const bool ok = sr >= 0 && k0 + c < K;
      cp_async_16(&As[st][r][c], ok ? a + (size_t)sr * lda + k0 + c : a, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {                  // W: 128 rows x 4 pieces of 8
      const int id = threadIdx.x + 256 * i;
      const int r = id >> 2, c = (id & 3) * 8;
      const bool ok = n0 + r < N && k0 + c < K;
      cp_async_16(&Ws[st][r][c], ok ? we + (size_t)(n0 + r) * K + k0 + c : we, ok);
    }
  };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp >> 2, wn = warp & 3;         // the warp's 32 x 32 part
  const int g = lane >> 2, t = lane & 3;
  float acc[2][4][4] = {};
  for (int s = 0; s < kTStages - 1; ++s) {
    if (s < nk) ask(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kb = 0; kb < nk; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kTStages - 2) : "memory");
    __syncthreads();                               // stage kb has landed; stage kb - 1 is free
    if (kb + kTStages - 1 < nk) ask(kb + kTStages - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int st = kb % kTStages;
#pragma unroll
    for (int kk = 0; kk < kTK; kk += 16) {
      uint32_t af[2][4], bfr[4][2];
      // ldmatrix: A 16 x 16 (lanes 0-15 the rows, lanes 16-31 the second 8 of k); B two column
      // tiles at once (lanes 0-7 / 8-15: the first tile's rows at k / k + 8, lanes 16-31 the second's)
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldsm_x4(af[i][0], af[i][1], af[i][2], af[i][3],
                &As[st][wm * 32 + i * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
      for (int jj = 0; jj < 2; ++jj)
        ldsm_x4(bfr[2 * jj][0], bfr[2 * jj][1], bfr[2 * jj + 1][0], bfr[2 * jj + 1][1],
                &Ws[st][wn * 32 + jj * 16 + (lane & 7) + ((lane >> 4) << 3)]
                   [kk + (((lane >> 3) & 1) << 3)]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bfr[j]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // c0, c1: row g, columns 2t, 2t + 1; c2, c3: row g + 8
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = wm * 32 + i * 16 + g + 8 * hh;
      if (r >= rows) continue;
      const size_t s = (size_t)(row0 + r);
      const float rw = (MODE == 2 && row_w) ? row_w[pair_of_pos[s]] : 1.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn * 32 + j * 8 + 2 * t;
        const float c0 = acc[i][j][2 * hh], c1 = acc[i][j][2 * hh + 1];
        if (MODE == 2) {
          __nv_bfloat16* out = (__nv_bfloat16*)out_ + s * N;
          const float u0 = fmaxf(to_f32(from_f32<__nv_bfloat16>(c0 * rw)), 0.f);
          const float u1 = fmaxf(to_f32(from_f32<__nv_bfloat16>(c1 * rw)), 0.f);
          if (n < N) out[n] = from_f32<__nv_bfloat16>(u0 * u0);
          if (n + 1 < N) out[n + 1] = from_f32<__nv_bfloat16>(u1 * u1);
        } else if (MODE == 1) {
          if (n < N) {
            const float gt = to_f32(from_f32<__nv_bfloat16>(c0)), up = to_f32(from_f32<__nv_bfloat16>(c1));
            ((__nv_bfloat16*)out_)[s * (N / 2) + n / 2] =
                from_f32<__nv_bfloat16>(clamped_glu(gt, up, limit, alpha, up_shift));
          }
        } else {
          float* out = (float*)out_ + s * N;
          if (n < N) out[n] = c0;
          if (n + 1 < N) out[n + 1] = c1;
        }
      }
    }
}

// ---- the same grouped products for a handful of pairs (decode steps of few requests) ------------
// There the work is the experts' weight bytes, and a tile of 64 rows that walks its whole reduction
// alone keeps too few of them under way (4 pairs: 45 us for 35 MB).  Here a tile is up to 8 rows of
// one expert, kept in shared memory; a block takes 16, 32 or 64 weight rows of that expert (the
// fewer pairs, the fewer rows, so that enough blocks keep loads under way), a warp two
// neighbouring rows at a time (a gate and its up value in the gated form), streamed once with
// 16-byte loads, each lane a strided share of the reduction, a warp sum at the end.  The order of
// the sums depends on K alone, so a pair's result does not depend on the batch.
constexpr int kFewRows = 8, kFewWarps = 8, kFewChunkMax = 64;

__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}

template <int MODE>
__global__ void __launch_bounds__(kFewWarps * 32)
moe_gemv_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w,
                int N, int K, const int* __restrict__ offsets, const int* __restrict__ pair_of_pos,
                int top, const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                const int* __restrict__ num_tiles, void* __restrict__ out_, float limit,
                float alpha, float up_shift, const float* __restrict__ row_w, int chunk) {
  extern __shared__ __align__(16) __nv_bfloat16 xrows[];           // [kFewRows][K]
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.x >= num_tiles[0]) return;
  const int e = tile_expert[blockIdx.x], row0 = tile_row0[blockIdx.x];
  const int rows = min(kFewRows, offsets[e + 1] - row0);
  const int k8 = K >> 3;
  for (int i = threadIdx.x; i < rows * k8; i += blockDim.x) {
    const int r = i / k8, c = (i - r * k8) * 8;
    const int src = MODE != 0 ? pair_of_pos[row0 + r] / top : row0 + r;
    *reinterpret_cast<uint4*>(xrows + (size_t)r * K + c) =
        *reinterpret_cast<const uint4*>(a + (size_t)src * lda + c);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* we = w + (size_t)e * N * K;
  for (int i = warp; i < chunk / 2; i += kFewWarps) {
    const int n = blockIdx.y * chunk + 2 * i;
    if (n >= N) break;                                             // N is even
    const __nv_bfloat16 *w0 = we + (size_t)n * K, *w1 = w0 + K;
    float acc0[kFewRows], acc1[kFewRows];
#pragma unroll
    for (int r = 0; r < kFewRows; ++r) acc0[r] = acc1[r] = 0.f;
    // four steps of the reduction at a time: their eight loads go out together, before any
    // arithmetic (left to the compiler, the loads of a step waited behind the branches of the
    // step before: 1.2 TB/s)
    for (int c0 = lane * 8; c0 < K; c0 += 4 * 256) {
      uint4 wa[4], wb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 256;
        if (c < K) {
          wa[u] = __ldg(reinterpret_cast<const uint4*>(w0 + c));
          wb[u] = __ldg(reinterpret_cast<const uint4*>(w1 + c));
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 256;
        if (c >= K) break;
        float f0[8], f1[8];
        bf16x8_to_f32(wa[u], f0);
        bf16x8_to_f32(wb[u], f1);
#pragma unroll
        for (int r = 0; r < kFewRows; ++r) {
          if (r < rows) {
            float x[8];
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(xrows + (size_t)r * K + c), x);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              acc0[r] = fmaf(f0[j], x[j], acc0[r]);
              acc1[r] = fmaf(f1[j], x[j], acc1[r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kFewRows; ++r) {
      if (r >= rows) break;                                        // uniform over the warp
      const float c0 = warp_sum(acc0[r]), c1 = warp_sum(acc1[r]);
      if (lane != 0) continue;
      const size_t s = (size_t)(row0 + r);
      if (MODE == 2) {
        const float rw = row_w ? row_w[pair_of_pos[s]] : 1.f;
        const float u0 = fmaxf(to_f32(from_f32<__nv_bfloat16>(c0 * rw)), 0.f);
        const float u1 = fmaxf(to_f32(from_f32<__nv_bfloat16>(c1 * rw)), 0.f);
        __nv_bfloat16* out = (__nv_bfloat16*)out_ + s * N + n;
        out[0] = from_f32<__nv_bfloat16>(u0 * u0);
        out[1] = from_f32<__nv_bfloat16>(u1 * u1);
      } else if (MODE == 1) {
        const float gt = to_f32(from_f32<__nv_bfloat16>(c0)), up = to_f32(from_f32<__nv_bfloat16>(c1));
        ((__nv_bfloat16*)out_)[s * (N / 2) + n / 2] =
            from_f32<__nv_bfloat16>(clamped_glu(gt, up, limit, alpha, up_shift));
      } else {
        float* out = (float*)out_ + s * N + n;
        out[0] = c0;
        out[1] = c1;
      }
    }
  }
}

// xs[s, :] = x[pair_of_pos[s] / top, :]: the tokens' rows in sorted order, 16 bytes an access, for
// the grouped product that reads its rows by TMA (K % 8 == 0, 16-byte aligned rows).
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                       const int* __restrict__ pair_of_pos, int top, int P, int K,
                                       __nv_bfloat16* __restrict__ xs) {
  pdl_trigger();
  pdl_wait();
  const int k8 = K >> 3;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)P * k8;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t s = i / k8;
    const int c = (int)(i - s * k8) * 8;
    const size_t src = (size_t)(pair_of_pos[s] / top) * ldx + c;
    *reinterpret_cast<uint4*>(xs + s * K + c) = *reinterpret_cast<const uint4*>(x + src);
  }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of_pair,
                                   const float* __restrict__ wgt, int top, int N,
                                   T* __restrict__ out) {
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(wgt ? wgt[(size_t)t * top + k] : 1.f,
                 y[(size_t)pos_of_pair[(size_t)t * top + k] * N + n], acc);
    out[(size_t)t * N + n] = from_f32<T>(acc);
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

// Rows of a tile: of the plain kernel (tensor_cores == 0) or of the tensor-core kernel.
GF_EXPORT int gf_moe_tile_rows(int tensor_cores) {
  return tensor_cores == 2 ? kFewRows : tensor_cores ? kTM : kBM;
}

// sigmoid != 0: a score is the sigmoid of its logit instead of the softmax over all experts.
GF_EXPORT int gf_moe_route(const float* logits, int T, int E, int top, int renorm, int sigmoid,
                           int* idx, float* wgt, void* stream) {
  if (T <= 0) return 0;
  if (E > kMaxExperts || top > E || top > 32) return -3;
  return launch_kernel(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                       logits, T, E, top, renorm, sigmoid, idx, wgt);
}

GF_EXPORT int gf_moe_plan(const int* idx, int P, int E, int tile_rows, int* offsets,
                          int* pos_of_pair, int* pair_of_pos, int* tile_expert, int* tile_row0,
                          int* num_tiles, void* stream) {
  if (P <= 0) return 0;
  if (E > kMaxExperts || tile_rows <= 0) return -3;
  return launch_kernel(moe_plan_kernel, dim3(E), dim3(kPlanThreads), 0, (cudaStream_t)stream, idx,
                       P, E, tile_rows, offsets, pos_of_pair, pair_of_pos, tile_expert, tile_row0,
                       num_tiles);
}

// first 1: gate/up product with the clamped GLU; out [P, N / 2] (dtype).  first 2: up product with
// relu(row_w * .)^2; out [P, N] (dtype); row_w [P] by pair, or null.  first 0: down; out fp32.
GF_EXPORT int gf_moe_gemm(const void* a, int lda, const void* w, int N, int K, const int* offsets,
                          const int* pair_of_pos, int top, const int* tile_expert,
                          const int* tile_row0, const int* num_tiles, int max_tiles, void* out,
                          int first, float limit, float alpha, float up_shift,
                          const float* row_w, int dtype, int tensor_cores, void* stream,
                          int pairs) {
  if (max_tiles <= 0) return 0;
  auto st = (cudaStream_t)stream;
  if (tensor_cores == 2) {                     // a handful of pairs: the weight-streaming kernel
    const size_t smem = (size_t)kFewRows * K * sizeof(bf);
    if (dtype != GF_BF16 || K % 8 || lda % 8 || N % 2 || (uintptr_t)a % 16 || (uintptr_t)w % 16 ||
        smem > 64 * 1024)
      return -3;
    // at most min(pairs, max_tiles) tiles hold rows; about four blocks an SM should be busy
    int chunk = kFewChunkMax;
    const int busy = pairs > 0 && pairs < max_tiles ? pairs : max_tiles;
    while (chunk > 2 * kFewWarps && (long long)busy * ((N + chunk - 1) / chunk) < 4 * 148) chunk /= 2;
    const dim3 fgrid(max_tiles, (N + chunk - 1) / chunk), fblock(kFewWarps * 32);
#define GF_FEW(MODE)                                                                              \
  {                                                                                               \
    static OncePerDevice attrs;                                                                   \
    if (int rc = attrs.run([&] {                                                                  \
          return cudaFuncSetAttribute(moe_gemv_kernel<MODE>,                                      \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);    \
        }))                                                                                       \
      return rc;                                                                                  \
    return launch_kernel(moe_gemv_kernel<MODE>, fgrid, fblock, smem, st, (const bf*)a, lda,        \
                         (const bf*)w, N, K, offsets, pair_of_pos, top, tile_expert, tile_row0,    \
                         num_tiles, out, limit, alpha, up_shift, row_w, chunk);                    \
  }
    if (first == 2) GF_FEW(2)
    if (first) GF_FEW(1)
    GF_FEW(0)
#undef GF_FEW
  }
  if (tensor_cores) {
    if (dtype != GF_BF16 || K % 8 || lda % 8 || (uintptr_t)a % 16 || (uintptr_t)w % 16) return -3;
    const dim3 tgrid(max_tiles, (N + kTN - 1) / kTN), tblock(256);
#define GF_TC(MODE)                                                                               \
  return launch_kernel(moe_gemm_mma_kernel<MODE>, tgrid, tblock, 0, st, (const bf*)a, lda,          \
                       (const bf*)w, N, K, offsets, pair_of_pos, top, tile_expert, tile_row0,       \
                       num_tiles, out, limit, alpha, up_shift, row_w)
    if (first == 2) GF_TC(2);
    if (first) GF_TC(1);
    GF_TC(0);
#undef GF_TC
  }
  const dim3 grid(max_tiles, (N + kBN - 1) / kBN), block(256);
#define GF_GO(T, MODE)                                                                           \
  return launch_kernel(moe_gemm_kernel<T, MODE>, grid, block, 0, st, (const T*)a, lda,           \
                       (const T*)w, N, K, offsets, pair_of_pos, top, tile_expert, tile_row0,      \
                       num_tiles, out, limit, alpha, up_shift, row_w)
  if (dtype == GF_F32) {
    if (first == 2) GF_GO(float, 2);
    if (first) GF_GO(float, 1);
    GF_GO(float, 0);
  }
  if (first == 2) GF_GO(bf, 2);
  if (first) GF_GO(bf, 1);
  GF_GO(bf, 0);
#undef GF_GO
}

GF_EXPORT int gf_moe_gather_rows(const void* x, int ldx, const int* pair_of_pos, int top, int P,
                                 int K, void* xs, void* stream) {
  if (P <= 0) return 0;
  if (K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15)) return -3;
  const size_t want = ((size_t)P * (K / 8) + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  return launch_kernel(moe_gather_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
                       (const bf*)x, ldx, pair_of_pos, top, P, K, (bf*)xs);
}

GF_EXPORT int gf_moe_combine(const float* y, const int* pos_of_pair, const float* wgt, int T,
                             int top, int N, void* out, int dtype, void* stream) {
  if (T <= 0) return 0;
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(moe_combine_kernel<float>, dim3(T), dim3(256), 0, st, y, pos_of_pair, wgt,
                         top, N, (float*)out);
  return launch_kernel(moe_combine_kernel<bf>, dim3(T), dim3(256), 0, st, y, pos_of_pair, wgt, top,
                       N, (bf*)out);
}
