// Routed feed-forward (mixture of experts): the router's choice, the regrouping of the step's tokens by expert,
// the experts' matrix products on the regrouped rows, and the weighted sum back into token order.
//
//  * moe_route: per token, s = softmax(router logits) over all experts in float32 (or, with `score` = 1, s = sigmoid of each logit
//    on its own); experts lie in `n_groups` equal
//    groups of neighbours, a group's score is its largest s (or the sum of its few largest), only the `keep` best groups stay eligible; the `top`
//    eligible experts with the largest s are chosen (ties: the lower index), each weighted s * route_scale, or
//    s / (sum of the chosen s) * route_scale with `renorm`. With a correction, groups and experts are chosen by s + correction[e]
//    and weighted by s alone.
//  * moe_sort: counts the (token, choice) pairs of every expert, lays the experts' rows out one after the other
//    (offsets[e] .. offsets[e + 1]) and gives every pair a row of its expert's range; tile_start[e] is the first tile of expert e.
//  * gemm_grouped: out[r] = W[e(r)] x[src(r)] for every regrouped row r: a 64 x 64 tile belongs to one expert; float32
//    FMA chains per output (a row's result does not depend on its place among the rows). With `gated`, W holds gate
//    rows then up rows and the output is silu(gate) * up.
//  * moe_combine: out[t] = sum_p base[p][t] + sum_k weight[t][k] * y[row(t, k)], in the order of the choices (without weights: the plain sum).
//  * scatter_scaled_rows: out[row(t, k)] = weight[t][k] * x[t]: the step's rows in the experts' order with the router's weight on the
//    expert's input (an expert is not linear, so a weight on its input is not one on its output).
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kRouteWarps = 4;

// (value, index) argmax over a warp: larger value wins, then the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int P, size_t stride_p, int T, int E, int n_groups, int keep, int top, float route_scale,
                                 int renorm, int* __restrict__ idx_out, float* __restrict__ wt_out, int score, const float* __restrict__ correction,
                                 int group_top) {
  // correction: a number per expert added to its score for the choice (of groups and of experts) and left out of the weights, or null.
  // group_top: a group's score is the sum of its `group_top` largest choice scores (1: its largest).
  // Choice scores may be negative: what cannot be chosen counts as minus infinity.
  extern __shared__ float sm[];   // per warp: E scores, E choice scores, then n_groups group scores
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= T) return;
  float* s = sm + (size_t)warp * (2 * E + n_groups);
  float* c = s + E;
  float* g = c + E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    float z = logits[(size_t)t * E + e];
    for (int p = 1; p < P; p++) z += logits[p * stride_p + (size_t)t * E + e];
    s[e] = z;
    mx = fmaxf(mx, z);
  }
  if (score == 1) {   // every expert's own sigmoid
    for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-s[e]));
  } else {
    mx = ib::warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(s[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = ib::warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) s[e] *= inv;
  }
  for (int e = lane; e < E; e += 32) c[e] = correction ? s[e] + correction[e] : s[e];
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int k = lane; k < n_groups; k += 32) {
      // the group's `group_top` largest choice scores, found one after the other (ties: the lower index first, which changes no sum)
      float total = 0.f;
      int taken[4] = {-1, -1, -1, -1};
      for (int r = 0; r < group_top && r < per; r++) {
        float b = -INFINITY;
        int bi = -1;
        for (int e = k * per; e < (k + 1) * per; e++) {
          if (e == taken[0] || e == taken[1] || e == taken[2] || e == taken[3]) continue;
          if (bi < 0 || c[e] > b) b = c[e], bi = e;
        }
        taken[r] = bi;
        total += b;
      }
      g[k] = total;
    }
    __syncwarp();
    for (int r = 0; r < keep; r++) {   // the best groups, one after the other; a kept group is marked in `g` by NaN
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int k = lane; k < n_groups; k += 32)
        if (g[k] == g[k] && (bi == 0x7fffffff || g[k] > bv)) bv = g[k], bi = k;
      warp_argmax(bv, bi);
      if (lane == 0 && bi < n_groups) g[bi] = __int_as_float(0x7fc00000);
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (g[e / per] == g[e / per]) c[e] = -INFINITY;   // its group was not kept
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int r = 0; r < top; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > bv) bv = c[e], bi = e;
    warp_argmax(bv, bi);
    float w = 0.f;
    if (bi >= E) bi = 0;   // fewer experts that can be chosen than choices: weight zero
    else w = s[bi];
    if (lane == 0) {
      idx_out[(size_t)t * top + r] = bi;
      wt_out[(size_t)t * top + r] = w;
      c[bi] = -INFINITY;
    }
    chosen_sum += w;
    __syncwarp();
  }
  if (lane == 0) {
    const float f = renorm ? route_scale / (chosen_sum > 0.f ? chosen_sum : 1.f) : route_scale;
    for (int r = 0; r < top; r++) wt_out[(size_t)t * top + r] *= f;
  }
}

constexpr int SM_ = 64;   // rows of a tile of the grouped product

__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int R, int top, int E, int tile_rows, int* __restrict__ offsets,
                                                        int* __restrict__ tile_start, int* __restrict__ row_of_pair, int* __restrict__ token_of_row) {
  extern __shared__ int si[];   // counts[E], fill[E], start[E + 1]
  int* counts = si;
  int* fill = si + E;
  int* start = si + 2 * E;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0, fill[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const int e = idx[r];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, tl = 0;
    for (int e = 0; e < E; e++) {
      start[e] = a;
      offsets[e] = a;
      tile_start[e] = tl;
      a += counts[e];
      tl += (counts[e] + tile_rows - 1) / tile_rows;
    }
    start[E] = a;
    offsets[E] = a;
    tile_start[E] = tl;
  }
  __syncthreads();
  // A pair takes the next free row of its expert's range. Which pair gets which row depends on the order threads run in; no result
  // does: every regrouped row is multiplied on its own, and the weighted sum goes back through row_of_pair in the order of the choices.
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const int e = idx[r];
    if (e < 0 || e >= E) continue;
    const int row = start[e] + atomicAdd(&fill[e], 1);
    row_of_pair[r] = row;
    token_of_row[row] = r / top;
  }
}

template <typename X, typename W, typename O>
__global__ void __launch_bounds__(256) gemm_grouped_kernel(const X* __restrict__ x, const int* __restrict__ src_row, const W* __restrict__ w,
                                                           O* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tile_start, int E,
                                                           int N, int K, int gated) {
  constexpr int BK = 16;
  __shared__ float xs[BK][SM_ + 1];
  __shared__ float ws[BK][64 + 1];
  __shared__ float us[BK][64 + 1];
  __shared__ int s_e, s_r0, s_r1;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  if (threadIdx.x == 0) {
    const int b = blockIdx.y;
    int e = -1;
    if (b < tile_start[E]) {
      int lo = 0, hi = E;   // the last e with tile_start[e] <= b
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= b) lo = mid;
        else hi = mid;
      }
      e = lo;
    }
    s_e = e;
    if (e >= 0) {
      s_r0 = offsets[e] + (b - tile_start[e]) * SM_;
      s_r1 = offsets[e + 1];
    }
  }
  __syncthreads();
  const int e = s_e;
  if (e < 0) return;
  const int r0 = s_r0, r1 = s_r1, n0 = blockIdx.x * 64;
  const int rows_w = gated ? 2 * N : N;
  const W* we = w + (size_t)e * rows_w * K;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[4][4], acu[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f, acu[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int idx = tid + q * 256, r = idx / BK, kk = idx % BK, k = k0 + kk;
      const int row = r0 + r, n = n0 + r;
      float xv = 0.f;
      if (row < r1 && k < K) {
        const int src = src_row ? src_row[row] : row;
        xv = ib::to_f32<X>(x[(size_t)src * K + k]);
      }
      xs[kk][r] = xv;
      ws[kk][r] = (n < N && k < K) ? ib::to_f32<W>(we[(size_t)n * K + k]) : 0.f;
      if (gated) us[kk][r] = (n < N && k < K) ? ib::to_f32<W>(we[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[4], c[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) c[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
      if (gated) {
#pragma unroll
        for (int j = 0; j < 4; j++) u[j] = us[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = r0 + ty * 4 + i;
    if (row >= r1) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (gated) {
        v = (v / (1.f + expf(-v))) * acu[i][j];
      }
      out[(size_t)row * N + n] = ib::from_f32<O>(v);
    }
  }
}

// out[r] = x[src_row[r]]: the step's rows in the experts' order (16 bytes a thread; K a multiple of 8).
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ src_row, uint4* __restrict__ out, int chunks) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.x;
  const uint4* src = x + (size_t)src_row[r] * chunks;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < chunks; c += gridDim.y * blockDim.x) out[(size_t)r * chunks + c] = src[c];
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair, const float* __restrict__ wt, int top,
                                   const float* __restrict__ base, int P, size_t stride_p, float* __restrict__ out, int H) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.y;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int p = 0; p < P; p++) a += base[p * stride_p + (size_t)t * H + i];
    if (wt) {
      for (int k = 0; k < top; k++) a = fmaf(wt[(size_t)t * top + k], y[(size_t)row_of_pair[(size_t)t * top + k] * H + i], a);
    } else {
      for (int k = 0; k < top; k++) a += y[(size_t)row_of_pair[(size_t)t * top + k] * H + i];
    }
    out[(size_t)t * H + i] = a;
  }
}

// out[row_of_pair[p]] = wt[p] * x[p / top] for every (token, choice) pair p; the product is taken in float32 and rounded once.
template <typename X>
__global__ void scatter_scaled_rows_kernel(const X* __restrict__ x, const int* __restrict__ row_of_pair, const float* __restrict__ wt, int top, X* __restrict__ out,
                                           int K) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int p = blockIdx.x;
  const float c = wt[p];
  const X* src = x + (size_t)(p / top) * K;
  X* dst = out + (size_t)row_of_pair[p] * K;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < K; i += gridDim.y * blockDim.x) dst[i] = ib::from_f32<X>(c * ib::to_f32<X>(src[i]));
}

}  // namespace

extern "C" int ib_moe_route(const float* logits, int P, long long stride_p, int T, int E, int n_groups, int keep, int top, float route_scale, int renorm,
                            int* idx_out, float* wt_out, int score, const float* correction, int group_top, cudaStream_t stream) {
  // correction: float32 [E] added to the scores for the choice only, or null; group_top: how many of a group's largest choice scores make its score (1 to 4).
  if (T == 0) return 0;
  IB_CHECK_ARG(group_top >= 1 && group_top <= 4, "moe_route: a group's score is the sum of its %d largest scores (1 to 4)", group_top);
  IB_CHECK_ARG(P >= 1 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes P=%d experts=%d top=%d", P, E, top);
  IB_CHECK_ARG(score == 0 || score == 1, "moe_route: score %d is neither 0 (softmax) nor 1 (sigmoid)", score);
  IB_CHECK_ARG(n_groups >= 1 && E % n_groups == 0 && keep >= 1 && keep <= n_groups, "moe_route: %d experts in %d groups of which %d stay", E, n_groups, keep);
  const size_t smem = (size_t)kRouteWarps * (2 * E + n_groups) * sizeof(float);
  IB_CHECK_ARG(smem <= 48 * 1024, "moe_route: %d experts need %zu bytes of shared memory, more than 48 KiB", E, smem);
  ib::launch(moe_route_kernel, (unsigned)((T + kRouteWarps - 1) / kRouteWarps), kRouteWarps * 32, smem, stream, logits, P, (size_t)stride_p, T, E, n_groups, keep,
             top, route_scale, renorm, idx_out, wt_out, score, correction, group_top);
  IB_CHECK_LAUNCH("moe_route");
  return 0;
}

extern "C" int ib_moe_tile_rows() { return SM_; }

// tile_rows: the rows of a tile of the product that will run on the regrouped rows (ib_moe_tile_rows() for this file's and the m16n8k16
// kernel; the token tile of the tcgen05 kernel).
extern "C" int ib_moe_sort(const int* idx, int R, int top, int E, int tile_rows, int* offsets, int* tile_start, int* row_of_pair, int* token_of_row,
                           cudaStream_t stream) {
  if (R == 0) return 0;
  IB_CHECK_ARG(R > 0 && top > 0 && E > 0 && tile_rows > 0, "moe_sort: bad sizes pairs=%d top=%d experts=%d tile=%d", R, top, E, tile_rows);
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  IB_CHECK_ARG(smem <= 48 * 1024, "moe_sort: %d experts need %zu bytes of shared memory, more than 48 KiB", E, smem);
  ib::launch(moe_sort_kernel, 1, 1024, smem, stream, idx, R, top, E, tile_rows, offsets, tile_start, row_of_pair, token_of_row);
  IB_CHECK_LAUNCH("moe_sort");
  return 0;
}

extern "C" int ib_gemm_grouped(const void* x, int x_dtype, const int* src_row, const void* w, int w_dtype, void* out, int out_dtype, const int* offsets,
                               const int* tile_start, int R, int E, int N, int K, int gated, cudaStream_t stream) {
  if (R == 0 || N == 0) return 0;
  IB_CHECK_ARG(R > 0 && E > 0 && N > 0 && K > 0, "gemm_grouped: bad sizes rows=%d experts=%d N=%d K=%d", R, E, N, K);
  dim3 grid((N + 63) / 64, R / SM_ + E);   // no more tiles than this, whatever the counts
  IB_CHECK_ARG(grid.y <= 65535, "gemm_grouped: %d rows exceed the grid limit", R);
  auto go = [&](auto kernel, auto* xp, auto* wp, auto* op) { ib::launch(kernel, grid, 256, 0, stream, xp, src_row, wp, op, offsets, tile_start, E, N, K, gated); };
  using bf = __nv_bfloat16;
  if (x_dtype == IB_F32 && w_dtype == IB_F32 && out_dtype == IB_F32) go(gemm_grouped_kernel<float, float, float>, (const float*)x, (const float*)w, (float*)out);
  else if (x_dtype == IB_BF16 && w_dtype == IB_BF16 && out_dtype == IB_F32) go(gemm_grouped_kernel<bf, bf, float>, (const bf*)x, (const bf*)w, (float*)out);
  else if (x_dtype == IB_BF16 && w_dtype == IB_BF16 && out_dtype == IB_BF16) go(gemm_grouped_kernel<bf, bf, bf>, (const bf*)x, (const bf*)w, (bf*)out);
  else return ib_set_error("gemm_grouped: unsupported dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
  IB_CHECK_LAUNCH("gemm_grouped");
  return 0;
}

extern "C" int ib_moe_combine(const float* y, const int* row_of_pair, const float* wt, int top, const float* base, int P, long long stride_p, float* out, int T,
                              int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && top > 0 && P >= 0, "moe_combine: bad sizes T=%d H=%d top=%d P=%d", T, H, top, P);
  IB_CHECK_ARG(T <= 65535, "moe_combine: T=%d rows exceed the grid limit 65535", T);
  dim3 grid(min((H + 255) / 256, 64), T);
  ib::launch(moe_combine_kernel, grid, 256, 0, stream, y, row_of_pair, wt, top, base, P, (size_t)stride_p, out, H);
  IB_CHECK_LAUNCH("moe_combine");
  return 0;
}

extern "C" int ib_gather_rows(const void* x, const int* src_row, void* out, int R, int K, int elem_bytes, cudaStream_t stream) {
  if (R == 0) return 0;
  IB_CHECK_ARG(R > 0 && K > 0 && (K * elem_bytes) % 16 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0), "gather_rows: rows of %d bytes must be multiples of 16, aligned",
               K * elem_bytes);
  const int chunks = K * elem_bytes / 16;
  ib::launch(gather_rows_kernel, dim3(R, min((chunks + 127) / 128, 8)), 128, 0, stream, (const uint4*)x, src_row, (uint4*)out, chunks);
  IB_CHECK_LAUNCH("gather_rows");
  return 0;
}

extern "C" int ib_scatter_scaled_rows(const void* x, int dtype, const int* row_of_pair, const float* wt, int top, void* out, int pairs, int K, cudaStream_t stream) {
  if (pairs == 0) return 0;
  IB_CHECK_ARG(pairs > 0 && K > 0 && top > 0, "scatter_scaled_rows: bad sizes pairs=%d K=%d top=%d", pairs, K, top);
  const dim3 grid((unsigned)pairs, (unsigned)min((K + 255) / 256, 8));
  if (dtype == IB_F32) ib::launch(scatter_scaled_rows_kernel<float>, grid, 256, 0, stream, (const float*)x, row_of_pair, wt, top, (float*)out, K);
  else if (dtype == IB_BF16)
    ib::launch(scatter_scaled_rows_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)x, row_of_pair, wt, top, (__nv_bfloat16*)out, K);
  else return ib_set_error("scatter_scaled_rows: unknown dtype %d", dtype);
  IB_CHECK_LAUNCH("scatter_scaled_rows");
  return 0;
}
