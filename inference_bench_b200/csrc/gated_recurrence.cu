// A gated linear recurrence with a matrix state per head (the HGRN2 form): for head a of a request, with q, f in R^D and v in R^V,
//     S <- diag(f) S + (1 - f) v^T,    o = S^T q,      f = lower + (1 - lower) * sigmoid(z_f + b_f),   q = silu(z_q)
// where z_q, z_f, v are the rows [q | f | v] of one fused projection (float32 partial sums, added in order). The state S [D, V] is
// float32, lives in the request's state slot, starts at zero and is carried from token to token; everything here is float32.
//
//  * gated_recurrence: one CTA per (segment, head, 32 or 16 value columns). A thread owns two neighbouring columns and RPT neighbouring rows of
//    S in registers; the tokens of the segment are walked in order, sixteen at a time: the CTA first turns the sixteen tokens' projections
//    into q, f and 1 - f in shared memory, then every thread updates its rows (the gates and queries of its rows come as 16-byte reads
//    and serve both columns) and adds its share of o, which a shuffle sums over the DS threads of the column pair. The kernel is bound by
//    instruction issue, not by memory: what counts is instructions per FMA. A decoded token is a segment of one: the cost is then the state's trip from memory and back.
//    With `chunks` the same kernel walks chunks of a long segment instead, each from a zero state: it leaves the chunk's own
//    outputs, its closing state and decay, and q_t times the decay from the chunk's start to t; `chunk_carry` then walks a segment's
//    chunks in order (S_in of the next = decay * S_in + the chunk's closing state, elementwise, ending in the request's state) and
//    `chunk_apply` adds (q_t * decay)^T S_in to every output. The three give what the walk over the whole segment gives, up to
//    rounding, with as many CTAs as the segment has chunks; which path a segment takes depends on its own length only.
//  * head_rmsnorm: out[t, a, :] = w * o[t, a, :] / sqrt(mean(o^2) + eps), into the activation dtype.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kChunk = 16;   // tokens prepared at a time

// RPT: rows of S a thread holds (for each of its two columns); kCols: value columns per CTA (32, or 16 where a thread holds sixteen rows)
template <int RPT, int kCols>
__global__ void __launch_bounds__(kCols * 16) gated_recurrence_kernel(const float* __restrict__ proj, int P, size_t stride_p, int R, const float* __restrict__ f_bias,
                                        const float* __restrict__ lower, float* __restrict__ state, size_t slot_stride, const int* __restrict__ seg_start,
                                        const int* __restrict__ seg_slot, float* __restrict__ o_out, int heads, int D, int V, int DS,
                                        const int* __restrict__ seg_list, const int* __restrict__ chunks, float* __restrict__ chunk_state,
                                        float* __restrict__ chunk_decay, float* __restrict__ qa_out, int form, int q_col, int f_col, int v_col) {
  // form 0: the gated form above (columns [q | f | v] at q_col, f_col, v_col of a row of R). form 1: a fixed decay per head and a key:
  // S <- lower[a] S + k v^T with q, k, v = silu of the columns at q_col, f_col, v_col (f_bias is not read; lower holds one decay a head).
  // seg_list: the segments this launch walks (null: all). chunks != null: blockIdx.x is a chunk (first row, rows) that starts from a zero
  // state and leaves its closing state in chunk_state[chunk][head], its decay in chunk_decay[chunk][head] and q * decay in qa_out[row][head].
  extern __shared__ float sm[];   // q[kChunk][D], f[kChunk][D], g[kChunk][D], v[kChunk][kCols], running decay [D]
  float* sq = sm;
  float* sf = sq + kChunk * D;
  float* sg = sf + kChunk * D;
  float* sv = sg + kChunk * D;
  float* run = sv + kChunk * kCols;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int a = blockIdx.y, j0 = blockIdx.z * kCols;
  const int tid = threadIdx.x, ds = tid % DS, col = 2 * (tid / DS), j = j0 + col;   // columns j and j + 1, rows ds * RPT .. ds * RPT + RPT - 1
  const int d0 = ds * RPT;
  const bool d4 = D % 4 == 0;
  int t0, t1;
  float* S;
  if (chunks) {
    t0 = chunks[2 * blockIdx.x];
    t1 = t0 + chunks[2 * blockIdx.x + 1];
    S = chunk_state + ((size_t)blockIdx.x * heads + a) * D * V;
    for (int d = tid; d < D; d += blockDim.x) run[d] = 1.f;
  } else {
    const int s = seg_list ? seg_list[blockIdx.x] : blockIdx.x;
    t0 = seg_start[s], t1 = seg_start[s + 1];
    S = state + (size_t)seg_slot[s] * slot_stride + (size_t)a * D * V;
  }
  float st[RPT][2];
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    const int d = d0 + r;
    st[r][0] = (!chunks && d < D && j < V) ? S[(size_t)d * V + j] : 0.f;
    st[r][1] = (!chunks && d < D && j + 1 < V) ? S[(size_t)d * V + j + 1] : 0.f;
  }
  const int q_off = q_col + a * D, f_off = f_col + a * D, v_off = v_col + a * V + j0;
  for (int c0 = t0; c0 < t1; c0 += kChunk) {
    const int n = min(kChunk, t1 - c0);
    __syncthreads();
    for (int i = tid; i < n * D; i += blockDim.x) {
      const int tt = i / D, d = i % D;
      const float* src = proj + (size_t)(c0 + tt) * R;
      float zq = src[q_off + d], zf = src[f_off + d];
      for (int p = 1; p < P; p++) zq += src[p * stride_p + q_off + d], zf += src[p * stride_p + f_off + d];
      sq[i] = zq / (1.f + expf(-zq));
      if (form == 1) {
        sf[i] = lower[a];
        sg[i] = zf / (1.f + expf(-zf));
      } else {
        zf += f_bias[a * D + d];
        const float lo = lower[a * D + d];
        const float sig = 1.f / (1.f + expf(-zf));
        const float f = __fmaf_rn(1.f - lo, sig, lo);
        sf[i] = f;
        sg[i] = 1.f - f;
      }
    }
    for (int i = tid; i < n * kCols; i += blockDim.x) {
      const int tt = i / kCols, c = i % kCols;
      float z = 0.f;
      if (j0 + c < V) {
        const float* src = proj + (size_t)(c0 + tt) * R + v_off + c;
        z = src[0];
        for (int p = 1; p < P; p++) z += src[p * stride_p];
        if (form == 1) z = z / (1.f + expf(-z));
      }
      sv[i] = z;
    }
    __syncthreads();
    if (chunks && blockIdx.z == 0) {   // q times the decay since the chunk's start, for the pass that adds the incoming state's share
      for (int d = tid; d < D; d += blockDim.x) {
        float r = run[d];
        for (int tt = 0; tt < n; tt++) {
          r *= sf[tt * D + d];
          qa_out[((size_t)(c0 + tt) * heads + a) * D + d] = sq[tt * D + d] * r;
        }
        run[d] = r;
      }
    }
    for (int tt = 0; tt < n; tt++) {
      const float v0 = sv[tt * kCols + col], v1 = sv[tt * kCols + col + 1];
      float f[RPT], g[RPT], q[RPT];
      if (d4 && d0 + RPT <= D) {   // this thread's rows are whole groups of four: 16-byte reads
#pragma unroll
        for (int r = 0; r < RPT; r += 4) {
          const float4 a = *(const float4*)(sf + tt * D + d0 + r), b = *(const float4*)(sg + tt * D + d0 + r), c = *(const float4*)(sq + tt * D + d0 + r);
          f[r] = a.x, f[r + 1] = a.y, f[r + 2] = a.z, f[r + 3] = a.w;
          g[r] = b.x, g[r + 1] = b.y, g[r + 2] = b.z, g[r + 3] = b.w;
          q[r] = c.x, q[r + 1] = c.y, q[r + 2] = c.z, q[r + 3] = c.w;
        }
      } else {
#pragma unroll
        for (int r = 0; r < RPT; r++) {
          const int d = d0 + r;
          const bool in = d < D;
          f[r] = in ? sf[tt * D + d] : 0.f, g[r] = in ? sg[tt * D + d] : 0.f, q[r] = in ? sq[tt * D + d] : 0.f;
        }
      }
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int r = 0; r < RPT; r++) {   // rows beyond D have f = g = q = 0: their state stays zero
        st[r][0] = __fmaf_rn(f[r], st[r][0], g[r] * v0);
        st[r][1] = __fmaf_rn(f[r], st[r][1], g[r] * v1);
        acc0 = __fmaf_rn(st[r][0], q[r], acc0);
        acc1 = __fmaf_rn(st[r][1], q[r], acc1);
      }
      for (int o = DS >> 1; o > 0; o >>= 1) {
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
      }
      if (ds == 0) {
        float* dst = o_out + ((size_t)(c0 + tt) * heads + a) * V + j;
        if (j < V) dst[0] = acc0;
        if (j + 1 < V) dst[1] = acc1;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    const int d = d0 + r;
    if (d < D && j < V) S[(size_t)d * V + j] = st[r][0];
    if (d < D && j + 1 < V) S[(size_t)d * V + j + 1] = st[r][1];
  }
  if (chunks && blockIdx.z == 0) {
    __syncthreads();
    for (int d = tid; d < D; d += blockDim.x) chunk_decay[((size_t)blockIdx.x * heads + a) * D + d] = run[d];
  }
}

// One thread per element (d, j) of a head's state walks a long segment's chunks in order: the chunk's place in chunk_state receives
// the state the chunk starts from, and the request's state slot the state after the last chunk.
__global__ void chunk_carry_kernel(const int* __restrict__ long_segs, const int* __restrict__ seg_slot, float* __restrict__ state, size_t slot_stride,
                                   float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int heads, int D, int V) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int s = long_segs[3 * blockIdx.x], c_first = long_segs[3 * blockIdx.x + 1], n_chunks = long_segs[3 * blockIdx.x + 2];
  const int a = blockIdx.y;
  float* S = state + (size_t)seg_slot[s] * slot_stride + (size_t)a * D * V;
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < D * V; e += gridDim.z * blockDim.x) {
    const int d = e / V;
    float cur = S[e];
    for (int c0 = c_first; c0 < c_first + n_chunks; c0 += 8) {   // eight chunks' values are requested before the first is used
      float own[8], dec[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int c = c0 + u;
        if (c < c_first + n_chunks) {
          own[u] = chunk_state[((size_t)c * heads + a) * D * V + e];
          dec[u] = chunk_decay[((size_t)c * heads + a) * D + d];
        }
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int c = c0 + u;
        if (c < c_first + n_chunks) {
          chunk_state[((size_t)c * heads + a) * D * V + e] = cur;
          cur = __fmaf_rn(dec[u], cur, own[u]);
        }
      }
    }
    S[e] = cur;
  }
}

// o[t][j] += sum_d qa[t][d] * S_in[d][j] for the rows of one chunk: a CTA of 256 threads takes 64 rows x 32 columns, 32 values of d at a time.
__global__ void __launch_bounds__(256) chunk_apply_kernel(const int* __restrict__ chunks, const float* __restrict__ chunk_state, const float* __restrict__ qa,
                                                          float* __restrict__ o_out, int heads, int D, int V) {
  __shared__ float s_in[32][33];
  __shared__ float s_q[64][33];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t0 = chunks[2 * blockIdx.x], n = chunks[2 * blockIdx.x + 1];
  const int a = blockIdx.y, j0 = blockIdx.z * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const float* Sin = chunk_state + ((size_t)blockIdx.x * heads + a) * D * V;
  float acc[8];
#pragma unroll
  for (int r = 0; r < 8; r++) acc[r] = 0.f;
  for (int d0 = 0; d0 < D; d0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * 32; i += 256) {
      const int dd = i >> 5, c = i & 31;
      s_in[dd][c] = (d0 + dd < D && j0 + c < V) ? Sin[(size_t)(d0 + dd) * V + j0 + c] : 0.f;
    }
    for (int i = threadIdx.x; i < 64 * 32; i += 256) {
      const int tt = i >> 5, dd = i & 31;
      s_q[tt][dd] = (tt < n && d0 + dd < D) ? qa[((size_t)(t0 + tt) * heads + a) * D + d0 + dd] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int dd = 0; dd < 32; dd++) {
      const float sv = s_in[dd][tx];
#pragma unroll
      for (int r = 0; r < 8; r++) acc[r] = __fmaf_rn(s_q[ty * 8 + r][dd], sv, acc[r]);
    }
  }
  if (j0 + tx < V) {
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const int tt = ty * 8 + r;
      if (tt < n) o_out[((size_t)(t0 + tt) * heads + a) * V + j0 + tx] += acc[r];
    }
  }
}

template <typename O>
__global__ void head_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, O* __restrict__ out, long long items, int V) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= items) return;
  const float* src = o + item * V;
  float ss = 0.f;
  for (int i = lane; i < V; i += 32) ss = __fmaf_rn(src[i], src[i], ss);
  const float inv = rsqrtf(ib::warp_sum(ss) / (float)V + eps);
  for (int i = lane; i < V; i += 32) out[item * V + i] = ib::from_f32<O>(w[i] * (src[i] * inv));
}

}  // namespace

// seg_list: int32 [n_segments] of the segments to walk (null: segments 0 .. n_segments - 1).
// chunks: null, or int32 [n_segments][2] = (first row, rows <= 64) of chunks that each start from a zero state (n_segments then counts
// chunks); chunk_state float32 [chunks][heads][D][V], chunk_decay float32 [chunks][heads][D] and qa float32 [T][heads][D] receive what
// ib_recurrence_chunks_finish needs.
extern "C" int ib_gated_recurrence(const float* proj, int P, long long stride_p, const float* f_bias, const float* lower, float* state, long long slot_stride,
                                   const int* seg_start, const int* seg_slot, int n_segments, float* o_out, int heads, int D, int V, const int* seg_list,
                                   const int* chunks, float* chunk_state, float* chunk_decay, float* qa, int form, int row, int q_col, int f_col, int v_col,
                                   cudaStream_t stream) {
  // form, row, q_col, f_col, v_col: see the kernel; row <= 0 stands for the gated form's own row [q | f | v] with its columns.
  if (n_segments == 0) return 0;
  IB_CHECK_ARG(form == 0 || form == 1, "gated_recurrence: form %d is not known (0: gated, 1: fixed decay with a key)", form);
  IB_CHECK_ARG(!chunks || (chunk_state && chunk_decay && qa), "gated_recurrence: chunks need their state, decay and query buffers");
  IB_CHECK_ARG(n_segments > 0 && P >= 1 && heads > 0 && D > 0 && V > 0, "gated_recurrence: bad sizes segments=%d P=%d heads=%d D=%d V=%d", n_segments, P, heads, D, V);
  IB_CHECK_ARG(D <= 512, "gated_recurrence: a head's key size %d is above 512", D);
  const int rpt = D <= 256 ? 8 : 16, kCols = D <= 256 ? 32 : 16;
  IB_CHECK_ARG(heads <= 65535 && (V + kCols - 1) / kCols <= 65535, "gated_recurrence: the grid is too large");
  int DS = 1;
  while (DS * rpt < D) DS *= 2;
  if (DS < 2) DS = 2;   // a CTA is a whole warp at least (kCols / 2 column pairs x DS)
  int R = 2 * heads * D + heads * V;
  if (row <= 0) q_col = 0, f_col = heads * D, v_col = 2 * heads * D;
  else R = row;
  IB_CHECK_ARG(q_col >= 0 && f_col >= 0 && v_col >= 0 && q_col + heads * D <= R && f_col + heads * D <= R && v_col + heads * V <= R,
               "gated_recurrence: the columns %d, %d, %d do not fit a row of %d", q_col, f_col, v_col, R);
  const size_t smem = ((size_t)kChunk * (3 * D + kCols) + D) * sizeof(float);
  const dim3 grid((unsigned)n_segments, (unsigned)heads, (unsigned)((V + kCols - 1) / kCols));
  auto go = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kCols / 2 * DS, smem, stream, proj, P, (size_t)stride_p, R, f_bias, lower, state, (size_t)slot_stride, seg_start, seg_slot, o_out, heads, D, V, DS,
               seg_list, chunks, chunk_state, chunk_decay, qa, form, q_col, f_col, v_col);
  };
  if (rpt == 8) go(gated_recurrence_kernel<8, 32>);
  else go(gated_recurrence_kernel<16, 16>);
  IB_CHECK_LAUNCH("gated_recurrence");
  return 0;
}

// After ib_gated_recurrence on chunks: long_segs int32 [n_long][3] = (segment, its first chunk, its chunks), chunks as above (n_chunks of them).
extern "C" int ib_recurrence_chunks_finish(const int* long_segs, int n_long, const int* chunks, int n_chunks, const int* seg_slot, float* state, long long slot_stride,
                                           float* chunk_state, const float* chunk_decay, const float* qa, float* o_out, int heads, int D, int V, cudaStream_t stream) {
  if (n_long == 0 || n_chunks == 0) return 0;
  IB_CHECK_ARG(n_long > 0 && n_chunks > 0 && heads > 0 && heads <= 65535 && D > 0 && V > 0, "recurrence_chunks_finish: bad sizes");
  ib::launch(chunk_carry_kernel, dim3((unsigned)n_long, (unsigned)heads, (unsigned)min((D * V + 255) / 256, 64)), 256, 0, stream, long_segs, seg_slot, state,
             (size_t)slot_stride, chunk_state, chunk_decay, heads, D, V);
  IB_CHECK_LAUNCH("recurrence chunk_carry");
  ib::launch(chunk_apply_kernel, dim3((unsigned)n_chunks, (unsigned)heads, (unsigned)((V + 31) / 32)), 256, 0, stream, chunks, (const float*)chunk_state, qa, o_out, heads, D, V);
  IB_CHECK_LAUNCH("recurrence chunk_apply");
  return 0;
}

extern "C" int ib_head_rmsnorm(const float* o, const float* w, float eps, void* out, int out_dtype, long long items, int V, cudaStream_t stream) {
  if (items == 0) return 0;
  IB_CHECK_ARG(items > 0 && V > 0, "head_rmsnorm: bad sizes items=%lld V=%d", items, V);
  const unsigned grid = (unsigned)((items + 3) / 4);
  if (out_dtype == IB_F32) ib::launch(head_rmsnorm_kernel<float>, grid, 128, 0, stream, o, w, eps, (float*)out, items, V);
  else if (out_dtype == IB_BF16) ib::launch(head_rmsnorm_kernel<__nv_bfloat16>, grid, 128, 0, stream, o, w, eps, (__nv_bfloat16*)out, items, V);
  else return ib_set_error("head_rmsnorm: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("head_rmsnorm");
  return 0;
}
