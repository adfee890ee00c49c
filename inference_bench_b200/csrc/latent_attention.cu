// Latent attention: every token leaves one row [c | kr] in the cache (a normed latent of `rank` values and one
// rotated key part of `rot` values that all heads share), and a head's keys and values are linear maps of c:
//   k_h = Wuk_h c,  v_h = Wuv_h c,  s = (q_nope . k_h + q_rope . kr) * scale,  o_h = sum_j p_j v_h,j.
// The kernels here work on the cached row directly (the maps are moved to the query and to the output):
//   q'_h = Wuk_h^T q_nope  (rank values),  s = ([q'_h | q_rope] . [c | kr]) * scale,  u_h = sum_j p_j c_j,  o_h = Wuv_h u_h,
// which is the same sum in another order, and reads rank + rot values a key instead of heads * (dim + vdim).
//
//  * latent_prepare: sums the split-K partial sums of the fused [q | dkv] projection; per head writes the unrotated
//    query part (activation dtype, the operand of the per-head product with Wuk) and the rotated part (float32, in
//    place in the full query row); norms the latent, rotates the shared key part and writes both to the cache.
//    Rotation pairs entry 2i with 2i + 1 (interleaved), angles from the step's cos/sin tables.
//  * gemm_heads: out[t][b][n] = sum_k x[t][b][k] w[b][n][k] for every head b (strided rows, FMA chains in float32):
//    the two per-head products above.
//  * latent_attention: a CTA per (token, eight heads, slice of the keys): key tiles of 32 rows go through shared memory
//    once for all heads of the CTA; a warp owns a head, a lane a key for the scores and output columns for the sum.
//    Scores, softmax weights and sums are float32. With slices, unnormalised partial results go to scratch and
//    latent_combine merges them.
#include <type_traits>

#include "kv_view.cuh"

namespace {

constexpr int kPrepWarps = 4;
constexpr int kAttnWarps = 8;
constexpr int kKeyTile = 32;

template <typename A, typename C>
__global__ void latent_prepare_kernel(const float* __restrict__ qd, int P, size_t stride_p, int row_len, const float* __restrict__ c_norm_w,
                                      float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half,
                                      const int* __restrict__ positions, const int* __restrict__ seg_of_token, A* __restrict__ q_nope,
                                      float* __restrict__ q_full, IbKvView kv, int write_kv, int T, int heads, int dim, int rot, int rank,
                                      unsigned* __restrict__ status) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = heads + (write_kv ? 1 : 0);
  const long long item = (long long)blockIdx.x * kPrepWarps + warp;
  if (item >= (long long)T * items) return;
  const int t = (int)(item / items), j = (int)(item % items);
  const float* row = qd + (size_t)t * row_len;
  auto summed = [&](int col) {
    float a = row[col];
    for (int p = 1; p < P; p++) a += row[p * stride_p + col];
    return a;
  };
  const float* cs = cos_t + (size_t)t * rot_half;
  const float* sn = sin_t + (size_t)t * rot_half;
  if (j < heads) {
    const int col0 = j * (dim + rot);
    A* qn = q_nope + ((size_t)t * heads + j) * dim;
    for (int d = lane; d < dim; d += 32) qn[d] = ib::from_f32<A>(summed(col0 + d));
    float* qr = q_full + ((size_t)t * heads + j) * (rank + rot) + rank;
    for (int i = lane; 2 * i < rot; i += 32) {
      const float a = summed(col0 + dim + 2 * i), b = 2 * i + 1 < rot ? summed(col0 + dim + 2 * i + 1) : 0.f;
      if (i < rot_half) {
        const float c = cs[i], s = sn[i];
        qr[2 * i] = a * c - b * s;
        if (2 * i + 1 < rot) qr[2 * i + 1] = b * c + a * s;
      } else {
        qr[2 * i] = a;
        if (2 * i + 1 < rot) qr[2 * i + 1] = b;
      }
    }
    return;
  }
  // the shared row: [rank latent values, normed | rot key values, rotated]
  const long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], 0);
  if (off < 0) {
    if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
    return;
  }
  C* dst = (C*)kv.base + off;
  const int col0 = heads * (dim + rot);
  float ss = 0.f;
  for (int d = lane; d < rank; d += 32) {
    const float a = summed(col0 + d);
    ss += a * a;
  }
  ss = ib::warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)rank + eps);
  for (int d = lane; d < rank; d += 32) dst[d] = ib::from_f32<C>(summed(col0 + d) * inv * c_norm_w[d]);
  for (int i = lane; 2 * i < rot; i += 32) {
    const float a = summed(col0 + rank + 2 * i), b = 2 * i + 1 < rot ? summed(col0 + rank + 2 * i + 1) : 0.f;
    float x = a, y = b;
    if (i < rot_half) {
      const float c = cs[i], s = sn[i];
      x = a * c - b * s;
      y = b * c + a * s;
    }
    dst[rank + 2 * i] = ib::from_f32<C>(x);
    if (2 * i + 1 < rot) dst[rank + 2 * i + 1] = ib::from_f32<C>(y);
  }
}

// The first product of a layer whose queries go through a latent of their own: [c_q raw (q_rank) | c raw (rank) | key part (rot) | ...].
// Per token, c_q is normed (weight w_q) into the activation dtype, the operand of the product that makes the heads' queries; the latent is
// normed, the shared key part rotated, and both written as the token's cache row. Further columns (gates) are left to their readers.
template <typename A, typename C>
__global__ void latent_down_kernel(const float* __restrict__ qd, int P, size_t stride_p, int row_len, int q_rank, const float* __restrict__ q_norm_w,
                                   A* __restrict__ cq, const float* __restrict__ c_norm_w, float eps, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int rot_half, const int* __restrict__ positions, const int* __restrict__ seg_of_token,
                                   IbKvView kv, int rank, int rot, unsigned* __restrict__ status) {
  // A CTA per token: the partial sums of the row's first q_rank + rank + rot columns are added once (several loads in flight) into shared
  // memory, the two sums of squares are block sums, and the threads then write the normed query latent and the cache row.
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x, n = q_rank + rank + rot;
  const float* src = qd + (size_t)t * row_len;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float a = src[i];
#pragma unroll 4
    for (int p = 1; p < P; p++) a += src[p * stride_p + i];
    row[i] = a;
    if (i < q_rank) sq = __fmaf_rn(a, a, sq);
    else if (i < q_rank + rank) sc = __fmaf_rn(a, a, sc);
  }
  sq = ib::block_sum(sq, scratch);
  sc = ib::block_sum(sc, scratch);
  const float inv_q = 1.f / sqrtf(sq / (float)q_rank + eps), inv_c = 1.f / sqrtf(sc / (float)rank + eps);
  for (int d = threadIdx.x; d < q_rank; d += blockDim.x) cq[(size_t)t * q_rank + d] = ib::from_f32<A>(row[d] * inv_q * q_norm_w[d]);
  const long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], 0);
  if (off < 0) {
    if (threadIdx.x == 0) atomicOr(status, IB_ERR_BAD_PAGE);
    return;
  }
  C* dst = (C*)kv.base + off;
  const float* c = row + q_rank;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = ib::from_f32<C>(c[d] * inv_c * c_norm_w[d]);
  const float* cs = cos_t + (size_t)t * rot_half;
  const float* sn = sin_t + (size_t)t * rot_half;
  for (int i = threadIdx.x; 2 * i < rot; i += blockDim.x) {
    const float a = c[rank + 2 * i], b = 2 * i + 1 < rot ? c[rank + 2 * i + 1] : 0.f;
    float x = a, y = b;
    if (i < rot_half) {
      const float co = cs[i], si = sn[i];
      x = a * co - b * si;
      y = b * co + a * si;
    }
    dst[rank + 2 * i] = ib::from_f32<C>(x);
    if (2 * i + 1 < rot) dst[rank + 2 * i + 1] = ib::from_f32<C>(y);
  }
}

// ---------------------------------------------------------------- per-head products
constexpr int GM = 64, GN = 64, GK = 16;

template <typename X, typename W, typename O>
__global__ void __launch_bounds__(256) gemm_heads_kernel(const X* __restrict__ x, long long x_row, long long x_head, const W* __restrict__ w,
                                                         O* __restrict__ out, long long o_row, long long o_head, int T, int N, int K,
                                                         const float* __restrict__ gate, int gate_P, size_t gate_stride, int gate_row) {
  // gate: float32 partial sums [gate_P][T][gate_row], offset to the first head's column, or null: head b's output of token t is multiplied by
  // the sigmoid of its column.
  __shared__ float xs[GK][GM + 1];
  __shared__ float ws[GK][GN + 1];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const X* xb = x + (size_t)b * x_head;
  const W* wb = w + (size_t)b * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int idx = tid + e * 256, r = idx / GK, kk = idx % GK, k = k0 + kk;
      const int t = t0 + r, n = n0 + r;
      xs[kk][r] = (t < T && k < K) ? ib::to_f32<X>(xb[(size_t)t * x_row + k]) : 0.f;
      ws[kk][r] = (n < N && k < K) ? ib::to_f32<W>(wb[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; kk++) {
      float a[4], c[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) c[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
    float f = 1.f;
    if (gate) {
      const float* gr = gate + (size_t)t * gate_row + b;
      float z = gr[0];
      for (int p = 1; p < gate_P; p++) z += gr[p * gate_stride];
      f = 1.f / (1.f + expf(-z));
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)t * o_row + (size_t)b * o_head + n] = ib::from_f32<O>(acc[i][j] * f);
    }
  }
}

// ---------------------------------------------------------------- attention over the cached rows
template <typename C, typename O, int NR>
__global__ void __launch_bounds__(kAttnWarps * 32) latent_attention_kernel(const float* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                                                           const int* __restrict__ seg_of_token, float scale, O* __restrict__ out,
                                                                           float* __restrict__ part_o, float* __restrict__ part_ml, int T, int H,
                                                                           int rank, int D, int n_slices, int slice_keys,
                                                                           unsigned* __restrict__ status, int window) {
  // window > 0: a token sees itself and the window - 1 positions before it; the slices then cut that range.
  extern __shared__ __align__(16) float smem[];
  __shared__ long long koff[kKeyTile];
  float* qs = smem;                          // [kAttnWarps][D]
  float* ks = smem + kAttnWarps * D;         // [kKeyTile][D + 1]
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y, h = blockIdx.x * kAttnWarps + warp, slice = blockIdx.z;
  const bool live = h < H;
  const int pos = positions[t], seg = seg_of_token[t];
  const int lo = (window > 0 ? max(0, pos - window + 1) : 0) + slice * slice_keys;
  const int hi = min(pos, lo + slice_keys - 1);   // last key of this slice (inclusive); lo > hi: nothing to see
  const int KS = D + 1;
  if (live) {
    const float* qrow = q + ((size_t)t * H + h) * D;
    for (int d = lane; d < D; d += 32) qs[warp * D + d] = qrow[d];
  }
  float acc[NR];
#pragma unroll
  for (int r = 0; r < NR; r++) acc[r] = 0.f;
  float m = -INFINITY, l = 0.f;
  const C* base = (const C*)kv.base;
  for (int k0 = lo; k0 <= hi; k0 += kKeyTile) {
    const int n = min(kKeyTile, hi - k0 + 1);
    __syncthreads();   // the tile before is no longer read (and qs is written)
    if (threadIdx.x < kKeyTile) {
      long long off = -1;
      if ((int)threadIdx.x < n) {
        off = ib::kv_offset(kv, seg, k0 + threadIdx.x, 0);
        if (off < 0) atomicOr(status, IB_ERR_BAD_PAGE);
      }
      koff[threadIdx.x] = off;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * D; idx += kAttnWarps * 32) {
      const int j = idx / D, d = idx - j * D;
      const long long off = koff[j];
      ks[j * KS + d] = off < 0 ? 0.f : ib::to_f32<C>(base[off + d]);
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < n && koff[lane] >= 0) {
      const float* kr = ks + lane * KS;
      const float* qw = qs + warp * D;
      float dot = 0.f;
      for (int d = 0; d < D; d++) dot = fmaf(qw[d], kr[d], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, ib::warp_max(s));
    if (m_new == -INFINITY) continue;
    const float corr = expf(m - m_new);
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    l = l * corr + ib::warp_sum(p);
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r] *= corr;
    for (int j = 0; j < n; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* kr = ks + j * KS;
#pragma unroll
      for (int r = 0; r < NR; r++) {
        const int d = lane + 32 * r;
        if (d < rank) acc[r] = fmaf(pj, kr[d], acc[r]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  if (n_slices == 1) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    O* o = out + ((size_t)t * H + h) * rank;
#pragma unroll
    for (int r = 0; r < NR; r++) {
      const int d = lane + 32 * r;
      if (d < rank) o[d] = ib::from_f32<O>(acc[r] * inv);
    }
    return;
  }
  const size_t unit = ((size_t)t * H + h) * n_slices + slice;
  float* po = part_o + unit * rank;
#pragma unroll
  for (int r = 0; r < NR; r++) {
    const int d = lane + 32 * r;
    if (d < rank) po[d] = acc[r];
  }
  if (lane == 0) {
    part_ml[2 * unit] = m;
    part_ml[2 * unit + 1] = l;
  }
}

template <typename O>
__global__ void latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, O* __restrict__ out, int rank,
                                      int n_slices) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const size_t unit0 = (size_t)blockIdx.x * n_slices;   // blockIdx.x = token * H + head
  float m = -INFINITY;
  for (int s = 0; s < n_slices; s++) m = fmaxf(m, part_ml[2 * (unit0 + s)]);
  float L = 0.f;
  for (int s = 0; s < n_slices; s++) {
    const float ms = part_ml[2 * (unit0 + s)];
    if (ms != -INFINITY) L += part_ml[2 * (unit0 + s) + 1] * expf(ms - m);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_slices; s++) {
      const float ms = part_ml[2 * (unit0 + s)];
      if (ms != -INFINITY) a = fmaf(part_o[(unit0 + s) * rank + d], expf(ms - m), a);
    }
    out[(size_t)blockIdx.x * rank + d] = ib::from_f32<O>(a * inv);
  }
}

int check_rows_view(const char* name, const IbKvView* kv) {
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "%s: the cache view has a null pointer", name);
  IB_CHECK_ARG(kv->kv_heads == 1 && kv->head_dim > 0, "%s: a latent cache has one row of head_dim values per token, got %d heads of %d", name,
               kv->kv_heads, kv->head_dim);
  IB_CHECK_ARG(kv->page_size > 0 && kv->num_pages > 0 && kv->table_stride > 0, "%s: bad page geometry", name);
  IB_CHECK_ARG(kv->dtype == IB_F32 || kv->dtype == IB_BF16, "%s: unknown cache dtype %d", name, kv->dtype);
  return 0;
}

}  // namespace

extern "C" int ib_latent_prepare(const float* qd, int P, long long stride_p, int row_len, const float* c_norm_w, float eps, const float* cos_t,
                                 const float* sin_t, int rot_half, const int* positions, const int* seg_of_token, void* q_nope, int act_dtype,
                                 float* q_full, const IbKvView* kv, int write_kv, int T, int heads, int dim, int rot, int rank, unsigned* status,
                                 cudaStream_t stream) {
  if (T == 0) return 0;
  if (check_rows_view("latent_prepare", kv)) return 1;
  IB_CHECK_ARG(P >= 1 && heads > 0 && dim >= 0 && rot >= 0 && rank > 0, "latent_prepare: bad sizes P=%d heads=%d dim=%d rot=%d rank=%d", P, heads, dim,
               rot, rank);
  IB_CHECK_ARG(kv->head_dim == rank + rot, "latent_prepare: the cache row has %d values, expected rank + rot = %d", kv->head_dim, rank + rot);
  IB_CHECK_ARG(2 * rot_half <= rot, "latent_prepare: %d rotated values exceed the rotated part of %d", 2 * rot_half, rot);
  IB_CHECK_ARG(row_len == heads * (dim + rot) + (write_kv ? rank + rot : 0), "latent_prepare: the projection has %d columns, expected %d", row_len,
               heads * (dim + rot) + (write_kv ? rank + rot : 0));
  IB_CHECK_ARG(!write_kv || c_norm_w, "latent_prepare: the latent's norm weight is missing");
  const long long items = (long long)T * (heads + (write_kv ? 1 : 0));
  const unsigned blocks = (unsigned)((items + kPrepWarps - 1) / kPrepWarps);
  auto go = [&](auto kernel, auto* qn) {
    ib::launch(kernel, blocks, kPrepWarps * 32, 0, stream, qd, P, (size_t)stride_p, row_len, c_norm_w, eps, cos_t, sin_t, rot_half, positions, seg_of_token,
               qn, q_full, *kv, write_kv, T, heads, dim, rot, rank, status);
  };
  if (act_dtype == IB_F32 && kv->dtype == IB_F32) go(latent_prepare_kernel<float, float>, (float*)q_nope);
  else if (act_dtype == IB_BF16 && kv->dtype == IB_BF16) go(latent_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, (__nv_bfloat16*)q_nope);
  else return ib_set_error("latent_prepare: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  IB_CHECK_LAUNCH("latent_prepare");
  return 0;
}

extern "C" int ib_latent_down(const float* qd, int P, long long stride_p, int row_len, int q_rank, const float* q_norm_w, void* cq, int act_dtype,
                              const float* c_norm_w, float eps, const float* cos_t, const float* sin_t, int rot_half, const int* positions,
                              const int* seg_of_token, const IbKvView* kv, int rank, int rot, int T, unsigned* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (check_rows_view("latent_down", kv)) return 1;
  IB_CHECK_ARG(P >= 1 && q_rank > 0 && rank > 0 && rot >= 0 && q_norm_w && c_norm_w && cq, "latent_down: bad sizes P=%d q_rank=%d rank=%d rot=%d", P, q_rank, rank, rot);
  IB_CHECK_ARG(kv->head_dim == rank + rot, "latent_down: the cache row has %d values, expected rank + rot = %d", kv->head_dim, rank + rot);
  IB_CHECK_ARG(2 * rot_half <= rot && row_len >= q_rank + rank + rot, "latent_down: a row of %d columns does not hold %d + %d + %d (turned: %d)", row_len, q_rank, rank,
               rot, 2 * rot_half);
  const size_t smem = (size_t)(q_rank + rank + rot) * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "latent_down: %d + %d + %d columns need %zu bytes of shared memory, more than 200 KiB", q_rank, rank, rot, smem);
  auto go = [&](auto kernel, auto* out) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, (unsigned)T, 128, smem, stream, qd, P, (size_t)stride_p, row_len, q_rank, q_norm_w, out, c_norm_w, eps, cos_t, sin_t, rot_half, positions,
               seg_of_token, *kv, rank, rot, status);
  };
  if (act_dtype == IB_F32 && kv->dtype == IB_F32) go(latent_down_kernel<float, float>, (float*)cq);
  else if (act_dtype == IB_BF16 && kv->dtype == IB_BF16) go(latent_down_kernel<__nv_bfloat16, __nv_bfloat16>, (__nv_bfloat16*)cq);
  else return ib_set_error("latent_down: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  IB_CHECK_LAUNCH("latent_down");
  return 0;
}

extern "C" int ib_gemm_heads(const void* x, int x_dtype, long long x_row, long long x_head, const void* w, int w_dtype, void* out, int out_dtype,
                             long long o_row, long long o_head, int T, int heads, int N, int K, const float* gate, int gate_P, long long gate_stride,
                             int gate_row, cudaStream_t stream) {
  // gate: float32 partial sums [gate_P][T][gate_row] offset to the first head's column (head b of token t is multiplied by the sigmoid of its column), or null.
  if (T == 0 || N == 0 || heads == 0) return 0;
  IB_CHECK_ARG(T > 0 && N > 0 && K > 0 && heads > 0, "gemm_heads: bad sizes T=%d heads=%d N=%d K=%d", T, heads, N, K);
  dim3 grid((N + GN - 1) / GN, (T + GM - 1) / GM, heads);
  IB_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "gemm_heads: T=%d or heads=%d exceed the grid limit", T, heads);
  auto go = [&](auto kernel, auto* xp, auto* wp, auto* op) { ib::launch(kernel, grid, 256, 0, stream, xp, x_row, x_head, wp, op, o_row, o_head, T, N, K, gate, gate_P, (size_t)gate_stride, gate_row); };
  using bf = __nv_bfloat16;
  if (x_dtype == IB_F32 && w_dtype == IB_F32 && out_dtype == IB_F32) go(gemm_heads_kernel<float, float, float>, (const float*)x, (const float*)w, (float*)out);
  else if (x_dtype == IB_BF16 && w_dtype == IB_BF16 && out_dtype == IB_F32) go(gemm_heads_kernel<bf, bf, float>, (const bf*)x, (const bf*)w, (float*)out);
  else if (x_dtype == IB_BF16 && w_dtype == IB_BF16 && out_dtype == IB_BF16) go(gemm_heads_kernel<bf, bf, bf>, (const bf*)x, (const bf*)w, (bf*)out);
  else return ib_set_error("gemm_heads: unsupported dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
  IB_CHECK_LAUNCH("gemm_heads");
  return 0;
}

extern "C" int ib_latent_attention_max_rank() { return 1024; }

// out[row] = the slices' unnormalised partial results of (token, head) `row`, merged and normalised.
extern "C" int ib_latent_combine(const float* part_o, const float* part_ml, void* out, int out_dtype, int rows, int rank, int n_slices, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (out_dtype == IB_F32) ib::launch(latent_combine_kernel<float>, (unsigned)rows, 128, 0, stream, part_o, part_ml, (float*)out, rank, n_slices);
  else if (out_dtype == IB_BF16) ib::launch(latent_combine_kernel<__nv_bfloat16>, (unsigned)rows, 128, 0, stream, part_o, part_ml, (__nv_bfloat16*)out, rank, n_slices);
  else return ib_set_error("latent_combine: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("latent_combine");
  return 0;
}

extern "C" int ib_latent_attention(const float* q, const IbKvView* kv, const int* positions, const int* seg_of_token, float scale, void* out,
                                   int out_dtype, float* part_o, float* part_ml, int T, int heads, int rank, int n_slices, int slice_keys,
                                   unsigned* status, int window, cudaStream_t stream) {
  if (T == 0) return 0;
  if (check_rows_view("latent_attention", kv)) return 1;
  const int D = kv->head_dim;
  IB_CHECK_ARG(heads > 0 && rank > 0 && rank <= D && rank <= 1024, "latent_attention: bad sizes heads=%d rank=%d row=%d (rank up to 1024)", heads, rank, D);
  IB_CHECK_ARG(n_slices >= 1 && slice_keys >= 1, "latent_attention: bad slicing %d x %d", n_slices, slice_keys);
  IB_CHECK_ARG(n_slices == 1 || (part_o && part_ml), "latent_attention: slices need scratch");
  IB_CHECK_ARG(T <= 65535 && n_slices <= 65535, "latent_attention: T=%d or slices=%d exceed the grid limit", T, n_slices);
  const size_t smem = ((size_t)kAttnWarps * D + (size_t)kKeyTile * (D + 1)) * sizeof(float);
  IB_CHECK_ARG(smem <= 220 * 1024, "latent_attention: a cache row of %d values needs %zu bytes of shared memory, more than 220 KiB", D, smem);
  dim3 grid((heads + kAttnWarps - 1) / kAttnWarps, T, n_slices);
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kAttnWarps * 32, smem, stream, q, *kv, positions, seg_of_token, scale, o, part_o, part_ml, T, heads, rank, D, n_slices, slice_keys,
               status, window);
  };
  auto pick = [&](auto c_tag, auto* o) {
    using C = decltype(c_tag);
    using O = std::remove_pointer_t<decltype(o)>;
    if (rank <= 64) go(latent_attention_kernel<C, O, 2>, o);
    else if (rank <= 128) go(latent_attention_kernel<C, O, 4>, o);
    else if (rank <= 256) go(latent_attention_kernel<C, O, 8>, o);
    else if (rank <= 512) go(latent_attention_kernel<C, O, 16>, o);
    else go(latent_attention_kernel<C, O, 32>, o);
  };
  if (out_dtype == IB_F32 && kv->dtype == IB_F32) pick(float(), (float*)out);
  else if (out_dtype == IB_BF16 && kv->dtype == IB_BF16) pick(__nv_bfloat16(), (__nv_bfloat16*)out);
  else return ib_set_error("latent_attention: output dtype %d and cache dtype %d must match", out_dtype, kv->dtype);
  IB_CHECK_LAUNCH("latent_attention");
  if (n_slices > 1) return ib_latent_combine(part_o, part_ml, out, out_dtype, T * heads, rank, n_slices, stream);
  return 0;
}
