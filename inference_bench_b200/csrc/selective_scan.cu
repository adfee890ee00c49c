// A selective state-space scan as a mixer's core (the Mamba form). Per channel c and state index n of a request, with x the output
// of a short causal convolution and SiLU, and [dt_low | B | C] = W_x x:
//     dt_c = softplus(W_dt[c] . dt_low + b_c)
//     S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c x_c B_n,      y_c = sum_n S[c][n] C_n + D_c x_c,      out_c = y_c * silu(z_c)
// S is float32, lives in the request's state slot, starts at zero and is carried from token to token; the step size, the exponentials
// and the sums are float32. The convolution's last taps - 1 inputs are the request's state as well (a second slot).
//
//  * conv_silu: x_t[c] = silu(b_c + sum_j w[j][c] u_(t - taps + 1 + j)[c]) where u are the rows of the input projection (float32 partial
//    sums, added in order) and rows before a segment's first token come from the request's convolution state. It only reads that state.
//  * selective_scan: one CTA per (segment, group of channels); G lanes share a channel and hold NPT states each in registers. Sixteen
//    tokens at a time are prepared in shared memory (dt_low, B, C summed from the projection's partial sums; the step sizes with their
//    small product, bias and softplus; x and z), then walked in order: the exponentials sit in the walk, everything else outside it.
//    The sum over a channel's states is a shuffle over its G lanes. After the walk the CTA writes the recurrent state and shifts the
//    request's convolution state (it runs after every reader of the old one).
//  * Long segments (prompt portions) are cut into chunks that are walked side by side. Since the decays of a channel's state n multiply
//    to exp(A[c][n] * sum of the chunk's step sizes), a chunk's effect on an incoming state is S_out = exp(A sum_dt) S_in + S_local:
//    pass 1 walks every chunk from a zero state and keeps S_local and sum_dt (no outputs), scan_chunks_carry walks a segment's chunks in
//    order for every (c, n), leaves each chunk's incoming state where its local one was, writes the request's state and shifts its
//    convolution state, and pass 2 walks every chunk again from its incoming state and writes the outputs.
#include "common.cuh"

namespace {

constexpr int kStage = 16;     // tokens prepared at a time
constexpr int kThreads = 128;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename O>
__global__ void conv_silu_kernel(const float* __restrict__ proj, int P, size_t stride_p, int R, const float* __restrict__ w, const float* __restrict__ bias, int taps,
                                 const float* __restrict__ conv_state, size_t slot_stride, const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                 const int* __restrict__ seg_slot, float* __restrict__ xc, O* __restrict__ xa, int inner) {
  // proj: [P][T][R], the convolution's inputs are its first `inner` columns; w: [taps][inner] (the last row is the current token's);
  // conv_state: [slots][taps - 1][inner]; xc: float32 [T][inner]; xa: the same in the activation dtype, or null.
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  const int s = seg_of_token[t], t0 = seg_start[s];
  const float* old = conv_state + (size_t)seg_slot[s] * slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < inner; c += gridDim.y * blockDim.x) {
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; j++) {
      const int u = t - (taps - 1) + j;
      float v;
      if (u >= t0) {
        const float* src = proj + (size_t)u * R + c;
        v = src[0];
        for (int p = 1; p < P; p++) v += src[p * stride_p];
      } else {
        v = old[(size_t)((taps - 1) + (u - t0)) * inner + c];
      }
      acc = __fmaf_rn(w[(size_t)j * inner + c], v, acc);
    }
    const float y = silu_f(acc);
    xc[(size_t)t * inner + c] = y;
    if (xa) xa[(size_t)t * inner + c] = ib::from_f32<O>(y);
  }
}

// The convolution's state of channel c becomes its inputs at the segment's last taps - 1 rows; with fewer rows than that the old state moves
// up. Row r is written after row r + n_seg was read, and later rows read only rows further on: in place, in rising order.
__device__ __forceinline__ void shift_conv_state(float* __restrict__ cs, const float* __restrict__ proj, int PZ, size_t z_stride, int RZ, int taps, int t0, int n_seg,
                                                 int inner, int c) {
  for (int r = 0; r < taps - 1; r++) {
    const int rel = n_seg - (taps - 1) + r;
    float v;
    if (rel >= 0) {
      const float* src = proj + (size_t)(t0 + rel) * RZ + c;
      v = src[0];
      for (int p = 1; p < PZ; p++) v += src[p * z_stride];
    } else {
      v = cs[(size_t)(n_seg + r) * inner + c];
    }
    cs[(size_t)r * inner + c] = v;
  }
}

template <int NPT, typename O>
__global__ void __launch_bounds__(kThreads) selective_scan_kernel(
    const float* __restrict__ xc, const float* __restrict__ low, int PL, size_t low_stride, const float* __restrict__ proj, int PZ, size_t z_stride, int RZ,
    const float* __restrict__ wdt, const float* __restrict__ dt_bias, const float* __restrict__ A, const float* __restrict__ Dv, float* __restrict__ state,
    size_t slot_stride, float* __restrict__ conv_state, size_t conv_slot_stride, int taps, const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
    O* __restrict__ out, int inner, int N, int rank, int G, const int* __restrict__ seg_list, const int* __restrict__ chunks, float* __restrict__ chunk_state,
    float* __restrict__ chunk_dt, int pass) {
  // pass 0: blockIdx.x is a segment (seg_list[blockIdx.x] if given), walked from and into the request's state. pass 1 and 2: blockIdx.x is
  // a chunk (chunks[b] = (first row, rows)); chunk_state: [chunks][inner][N], chunk_dt: [chunks][inner].
  // low: [PL][T][rank + 2N] = [dt_low | B | C]; proj: [PZ][T][RZ] = [u | z] (u: the convolution's inputs, z at column `inner`);
  // wdt: float32 [inner][rank]; A: float32 [inner][N], already -exp(A_log); state: [slots][inner][N]; out: [T][inner].
  extern __shared__ float sm[];
  const int CH = kThreads / G, RL = rank + 2 * N, WS = rank + 1;
  float* s_w = sm;                       // [CH][rank + 1]
  float* s_low = s_w + CH * WS;          // [kStage][RL]
  float* s_dt = s_low + kStage * RL;     // [kStage][CH]
  float* s_x = s_dt + kStage * CH;
  float* s_z = s_x + kStage * CH;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int c_first = blockIdx.y * CH;
  const int tid = threadIdx.x, cl = tid / G, g = tid % G, c = c_first + cl;
  const int s = pass ? 0 : (seg_list ? seg_list[blockIdx.x] : (int)blockIdx.x);
  const int t0 = pass ? chunks[2 * blockIdx.x] : seg_start[s], t1 = pass ? t0 + chunks[2 * blockIdx.x + 1] : seg_start[s + 1];
  const bool live = c < inner;
  float* S = pass ? chunk_state + ((size_t)blockIdx.x * inner + c) * N : state + (size_t)seg_slot[s] * slot_stride + (size_t)c * N;
  float st[NPT], a[NPT];
#pragma unroll
  for (int i = 0; i < NPT; i++) {
    const int n = g + i * G;
    const bool in = live && n < N;
    st[i] = in && pass != 1 ? S[n] : 0.f;
    a[i] = in ? A[(size_t)c * N + n] : 0.f;
  }
  float dt_sum = 0.f;
  for (int i = tid; i < CH * rank; i += kThreads) {
    const int cc = i / rank, r = i % rank;
    s_w[cc * WS + r] = c_first + cc < inner ? wdt[(size_t)(c_first + cc) * rank + r] : 0.f;
  }
  const float d_skip = live ? Dv[c] : 0.f;
  for (int b0 = t0; b0 < t1; b0 += kStage) {
    const int n_tok = min(kStage, t1 - b0);
    __syncthreads();
    for (int i = tid; i < n_tok * RL; i += kThreads) {
      const int tt = i / RL, r = i % RL;
      const float* src = low + (size_t)(b0 + tt) * RL + r;
      float v = src[0];
      for (int p = 1; p < PL; p++) v += src[p * low_stride];
      s_low[i] = v;
    }
    for (int i = tid; i < n_tok * CH; i += kThreads) {
      const int tt = i / CH, cc = i % CH;
      float xv = 0.f, zv = 0.f;
      if (c_first + cc < inner) {
        xv = xc[(size_t)(b0 + tt) * inner + c_first + cc];
        if (pass != 1) {
          const float* src = proj + (size_t)(b0 + tt) * RZ + inner + c_first + cc;
          zv = src[0];
          for (int p = 1; p < PZ; p++) zv += src[p * z_stride];
        }
      }
      s_x[i] = xv;
      s_z[i] = zv;
    }
    __syncthreads();
    for (int i = tid; i < n_tok * CH; i += kThreads) {
      const int tt = i / CH, cc = i % CH;
      float acc = c_first + cc < inner ? dt_bias[c_first + cc] : 0.f;
      for (int r = 0; r < rank; r++) acc = __fmaf_rn(s_low[tt * RL + r], s_w[cc * WS + r], acc);
      s_dt[i] = softplus_f(acc);
    }
    __syncthreads();
    for (int tt = 0; tt < n_tok; tt++) {
      const float dtv = s_dt[tt * CH + cl], xv = s_x[tt * CH + cl];
      const float dx = dtv * xv;
      const float* bc = s_low + tt * RL + rank;
      float acc = 0.f;
      if (pass == 1) {
        dt_sum += dtv;
#pragma unroll
        for (int i = 0; i < NPT; i++) {
          const int n = g + i * G;
          st[i] = __fmaf_rn(expf(dtv * a[i]), st[i], dx * (n < N ? bc[n] : 0.f));
        }
        continue;
      }
#pragma unroll
      for (int i = 0; i < NPT; i++) {
        const int n = g + i * G;
        const float bn = n < N ? bc[n] : 0.f, cn = n < N ? bc[N + n] : 0.f;
        st[i] = __fmaf_rn(expf(dtv * a[i]), st[i], dx * bn);
        acc = __fmaf_rn(st[i], cn, acc);
      }
      for (int o = G >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (g == 0 && live) {
        const float y = __fmaf_rn(d_skip, xv, acc);
        out[(size_t)(b0 + tt) * inner + c] = ib::from_f32<O>(y * silu_f(s_z[tt * CH + cl]));
      }
    }
  }
  if (pass == 2) return;
#pragma unroll
  for (int i = 0; i < NPT; i++) {
    const int n = g + i * G;
    if (live && n < N) S[n] = st[i];
  }
  if (pass == 1) {
    if (g == 0 && live) chunk_dt[(size_t)blockIdx.x * inner + c] = dt_sum;
    return;
  }
  if (g == 0 && live && taps > 1)
    shift_conv_state(conv_state + (size_t)seg_slot[s] * conv_slot_stride, proj, PZ, z_stride, RZ, taps, t0, t1 - t0, inner, c);
}

__global__ void scan_chunks_carry_kernel(const int* __restrict__ long_segs, const int* __restrict__ seg_start, const int* __restrict__ seg_slot, float* __restrict__ state,
                                         size_t slot_stride, float* __restrict__ chunk_state, const float* __restrict__ chunk_dt, const float* __restrict__ A,
                                         const float* __restrict__ proj, int PZ, size_t z_stride, int RZ, float* __restrict__ conv_state, size_t conv_slot_stride,
                                         int taps, int inner, int N) {
  // long_segs: [n][3] = (segment, first chunk, chunks). One thread per (channel, state index) walks the segment's chunks in order: the
  // chunk's local state gives way to its incoming one, and the request's state becomes the last chunk's outgoing one.
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int s = long_segs[3 * blockIdx.x], first = long_segs[3 * blockIdx.x + 1], count = long_segs[3 * blockIdx.x + 2];
  const size_t per = (size_t)inner * N;
  for (size_t i = (size_t)blockIdx.y * blockDim.x + threadIdx.x; i < per; i += (size_t)gridDim.y * blockDim.x) {
    const int c = (int)(i / N);
    float* S = state + (size_t)seg_slot[s] * slot_stride + i;
    const float a = A[i];
    float v = *S;
    for (int k = first; k < first + count; k++) {
      float* loc = chunk_state + (size_t)k * per + i;
      const float mine = *loc;
      *loc = v;
      v = __fmaf_rn(expf(a * chunk_dt[(size_t)k * inner + c]), v, mine);
    }
    *S = v;
    if (i % N == 0 && taps > 1)
      shift_conv_state(conv_state + (size_t)seg_slot[s] * conv_slot_stride, proj, PZ, z_stride, RZ, taps, seg_start[s], seg_start[s + 1] - seg_start[s], inner, c);
  }
}

}  // namespace

extern "C" int ib_conv_silu(const float* proj, int P, long long stride_p, int R, const float* w, const float* bias, int taps, const float* conv_state,
                            long long slot_stride, const int* seg_of_token, const int* seg_start, const int* seg_slot, float* xc, void* xa, int act_dtype, int T,
                            int inner, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && inner > 0 && P >= 1 && taps >= 1 && R >= inner, "conv_silu: bad sizes T=%d inner=%d P=%d taps=%d R=%d", T, inner, P, taps, R);
  const dim3 grid((unsigned)T, (unsigned)min((inner + 255) / 256, 64));
  if (!xa || act_dtype == IB_F32)
    ib::launch(conv_silu_kernel<float>, grid, 256, 0, stream, proj, P, (size_t)stride_p, R, w, bias, taps, conv_state, (size_t)slot_stride, seg_of_token, seg_start,
               seg_slot, xc, (float*)xa, inner);
  else if (act_dtype == IB_BF16)
    ib::launch(conv_silu_kernel<__nv_bfloat16>, grid, 256, 0, stream, proj, P, (size_t)stride_p, R, w, bias, taps, conv_state, (size_t)slot_stride, seg_of_token,
               seg_start, seg_slot, xc, (__nv_bfloat16*)xa, inner);
  else
    return ib_set_error("conv_silu: unknown activation dtype %d", act_dtype);
  IB_CHECK_LAUNCH("conv_silu");
  return 0;
}

extern "C" int ib_selective_scan(const float* xc, const float* low, int PL, long long low_stride, const float* proj, int PZ, long long z_stride, int RZ, const float* wdt,
                                 const float* dt_bias, const float* A, const float* Dv, float* state, long long slot_stride, float* conv_state,
                                 long long conv_slot_stride, int taps, const int* seg_start, const int* seg_slot, int n_segments, void* out, int out_dtype, int inner,
                                 int N, int rank, const int* seg_list, const int* chunks, float* chunk_state, float* chunk_dt, int pass, cudaStream_t stream) {
  // n_segments: the grid's first extent, that is segments (pass 0; those of seg_list if given) or chunks (pass 1 and 2).
  if (n_segments == 0) return 0;
  IB_CHECK_ARG(pass >= 0 && pass <= 2 && (pass == 0 || (chunks && chunk_state && chunk_dt)), "selective_scan: pass %d needs the chunk table and its buffers", pass);
  IB_CHECK_ARG(n_segments > 0 && inner > 0 && N > 0 && rank > 0 && PL >= 1 && PZ >= 1 && taps >= 1, "selective_scan: bad sizes segments=%d inner=%d N=%d rank=%d", n_segments,
               inner, N, rank);
  IB_CHECK_ARG(N <= 256, "selective_scan: %d states a channel are above the 256 the kernel holds", N);
  IB_CHECK_ARG(RZ >= 2 * inner, "selective_scan: the input projection's row of %d is shorter than 2 x %d", RZ, inner);
  const int npt = N <= 128 ? 4 : 8;
  int G = 1;
  while (G * npt < N) G *= 2;
  const int CH = kThreads / G;
  const size_t smem = ((size_t)CH * (rank + 1) + (size_t)kStage * (rank + 2 * N) + 3 * (size_t)kStage * CH) * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "selective_scan: dt_rank %d and %d states need %zu bytes of shared memory, more than 200 KiB", rank, N, smem);
  const dim3 grid((unsigned)n_segments, (unsigned)((inner + CH - 1) / CH));
  IB_CHECK_ARG(grid.y <= 65535, "selective_scan: the grid is too large");
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kThreads, smem, stream, xc, low, PL, (size_t)low_stride, proj, PZ, (size_t)z_stride, RZ, wdt, dt_bias, A, Dv, state, (size_t)slot_stride,
               conv_state, (size_t)conv_slot_stride, taps, seg_start, seg_slot, o, inner, N, rank, G, seg_list, chunks, chunk_state, chunk_dt, pass);
  };
  if (out_dtype == IB_F32) {
    if (npt == 4) go(selective_scan_kernel<4, float>, (float*)out);
    else go(selective_scan_kernel<8, float>, (float*)out);
  } else if (out_dtype == IB_BF16) {
    if (npt == 4) go(selective_scan_kernel<4, __nv_bfloat16>, (__nv_bfloat16*)out);
    else go(selective_scan_kernel<8, __nv_bfloat16>, (__nv_bfloat16*)out);
  } else {
    return ib_set_error("selective_scan: unknown output dtype %d", out_dtype);
  }
  IB_CHECK_LAUNCH("selective_scan");
  return 0;
}

extern "C" int ib_scan_chunks_carry(const int* long_segs, int n_long, const int* seg_start, const int* seg_slot, float* state, long long slot_stride, float* chunk_state,
                                    const float* chunk_dt, const float* A, const float* proj, int PZ, long long z_stride, int RZ, float* conv_state,
                                    long long conv_slot_stride, int taps, int inner, int N, cudaStream_t stream) {
  if (n_long == 0) return 0;
  IB_CHECK_ARG(n_long > 0 && inner > 0 && N > 0 && taps >= 1 && PZ >= 1, "scan_chunks_carry: bad sizes segments=%d inner=%d N=%d taps=%d", n_long, inner, N, taps);
  const dim3 grid((unsigned)n_long, (unsigned)min(((size_t)inner * N + 255) / 256, (size_t)4096));
  ib::launch(scan_chunks_carry_kernel, grid, 256, 0, stream, long_segs, seg_start, seg_slot, state, (size_t)slot_stride, chunk_state, chunk_dt, A, proj, PZ,
             (size_t)z_stride, RZ, conv_state, (size_t)conv_slot_stride, taps, inner, N);
  IB_CHECK_LAUNCH("scan_chunks_carry");
  return 0;
}
