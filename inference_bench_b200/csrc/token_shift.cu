// Row-wise kernels around a token shift, a loop over layers, a gated norm over all heads and a two-sided quadratic/exponential
// activation. All arithmetic is float32; only a stored activation may be bfloat16.
//
//  * token_shift_rows: out_t = h_t + (h_(t-1) - h_t) * mix per channel, with h as it was before the replacement. The row before a
//    segment's first row is the request's state (zeros at admission); the segment's last row becomes the new state. The CTA that reads
//    a request's old state is the one that writes the new one (the first row's), each thread for the channels it read.
//  * add_rmsnorm_shift_single: for a step whose segments all bring one token: the residual add (partial sums in order, an optional bias),
//    the RMS norm and the shift in one kernel; the normed row never leaves the CTA.
//  * add_rmsnorm_bias: the residual add with a bias and the norm, for the norms that follow a mixer whose output has a bias.
//  * loop_pack: before a pass over looped layers: packed_t = [x_t + pending | x0_t] in the activation dtype (the input of the matrix
//    that makes the pass's stream) and x_t = step vector, to which the next norm adds the product.
//  * xielu_rows: act = z > 0 ? ap z^2 + z / 2 : an (exp(z) - 1 - z) + z / 2 with ap = softplus(p), an = 1/2 + softplus(q).
//  * gated_rmsnorm: out = scale * w * o / sqrt(mean(o^2) + eps) * sigmoid(gate) over a whole row of all heads.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

template <typename O>
__global__ void token_shift_rows_kernel(const float* __restrict__ h, const float* __restrict__ mix, float* __restrict__ state, size_t slot_stride,
                                        const int* __restrict__ seg_of_token, const int* __restrict__ seg_start, const int* __restrict__ seg_slot, O* __restrict__ out,
                                        int H) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  const int s = seg_of_token[t], t0 = seg_start[s];
  const bool first = t == t0;
  float* st = state + (size_t)seg_slot[s] * slot_stride;
  const float* prev = first ? st : h + (size_t)(t - 1) * H;
  const float* last = h + (size_t)(seg_start[s + 1] - 1) * H;
  const float* cur = h + (size_t)t * H;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
    const float v = cur[i], p = prev[i];
    out[(size_t)t * H + i] = ib::from_f32<O>(__fmaf_rn(p - v, mix[i], v));
    if (first) st[i] = last[i];
  }
}

// One CTA per row. SHIFT: row t is segment t; the state is read and replaced by the same thread.
template <typename O, bool SHIFT>
__global__ void add_rmsnorm_ext_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride, const float* __restrict__ bias,
                                       const float* __restrict__ w, float eps, const float* __restrict__ mix, float* __restrict__ state, size_t slot_stride,
                                       const int* __restrict__ seg_slot, O* __restrict__ out, int H) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = xr[i];
    if (P > 0) {
      const float* dr = delta + (size_t)t * H + i;
      float d = dr[0];
      for (int p = 1; p < P; p++) d += dr[p * delta_stride];
      if (bias) d += bias[i];
      v += d;
      xr[i] = v;
    }
    row[i] = v;
    ss = __fmaf_rn(v, v, ss);
  }
  ss = ib::block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  float* st = SHIFT ? state + (size_t)seg_slot[t] * slot_stride : nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = w[i] * (row[i] * inv);
    if constexpr (SHIFT) {
      const float p = st[i];
      st[i] = v;
      v = __fmaf_rn(p - v, mix[i], v);
    }
    out[(size_t)t * H + i] = ib::from_f32<O>(v);
  }
}

template <typename O>
__global__ void loop_pack_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride, const float* __restrict__ x0,
                                 const float* __restrict__ step, O* __restrict__ packed, int H) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
    float v = x[(size_t)t * H + i];
    if (P > 0) {
      const float* dr = delta + (size_t)t * H + i;
      float d = dr[0];
      for (int p = 1; p < P; p++) d += dr[p * delta_stride];
      v += d;
    }
    packed[(size_t)t * 2 * H + i] = ib::from_f32<O>(v);
    packed[(size_t)t * 2 * H + H + i] = ib::from_f32<O>(x0[(size_t)t * H + i]);
    x[(size_t)t * H + i] = step[i];
  }
}

__global__ void add_bias_rows_kernel(float* __restrict__ v, const float* __restrict__ bias, int H) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) v[(size_t)t * H + i] += bias[i];
}

template <typename O>
__global__ void xielu_rows_kernel(const float* __restrict__ z, int P, size_t stride, const float* __restrict__ pq, O* __restrict__ act, int I) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.y;
  const float ap = ib::softplus(pq[0]), an = 0.5f + ib::softplus(pq[1]);
  const float* row = z + (size_t)t * I;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I; i += gridDim.x * blockDim.x) {
    float v = row[i];
    for (int p = 1; p < P; p++) v += row[p * stride + i];
    act[(size_t)t * I + i] = ib::from_f32<O>(ib::xielu(v, ap, an));
  }
}

template <typename O>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const float* __restrict__ gate, int P, size_t gate_stride,
                                     int gate_row, float scale, O* __restrict__ out, int out_row, int H) {
  // o: [T][H]; gate: partial sums [P][T][gate_row], already offset to the gate's first column; out: rows of out_row values, offset to the first column
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int t = blockIdx.x;
  const float* src = o + (size_t)t * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ss = __fmaf_rn(src[i], src[i], ss);
  ss = ib::block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float* gr = gate + (size_t)t * gate_row + i;
    float g = gr[0];
    for (int p = 1; p < P; p++) g += gr[p * gate_stride];
    out[(size_t)t * out_row + i] = ib::from_f32<O>(scale * (w[i] * (src[i] * inv)) * sigmoid_f(g));
  }
}

int row_threads(int H) { return H >= 4096 ? 1024 : (H >= 1024 ? 512 : 256); }

}  // namespace

extern "C" int ib_token_shift_rows(const float* h, const float* mix, float* state, long long slot_stride, const int* seg_of_token, const int* seg_start,
                                   const int* seg_slot, void* out, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0, "token_shift_rows: bad sizes T=%d H=%d", T, H);
  const dim3 grid((unsigned)T, (unsigned)min((H + 255) / 256, 64));
  if (out_dtype == IB_F32) ib::launch(token_shift_rows_kernel<float>, grid, 256, 0, stream, h, mix, state, (size_t)slot_stride, seg_of_token, seg_start, seg_slot, (float*)out, H);
  else if (out_dtype == IB_BF16)
    ib::launch(token_shift_rows_kernel<__nv_bfloat16>, grid, 256, 0, stream, h, mix, state, (size_t)slot_stride, seg_of_token, seg_start, seg_slot, (__nv_bfloat16*)out, H);
  else return ib_set_error("token_shift_rows: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("token_shift_rows");
  return 0;
}

// mix == null: the residual add (with an optional bias) and the norm; otherwise also the shift, for a step whose row t is segment t.
extern "C" int ib_add_rmsnorm_ext(float* x, const float* delta, int P, long long delta_stride, const float* bias, const float* w, float eps, const float* mix,
                                  float* state, long long slot_stride, const int* seg_slot, void* out, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && P >= 0 && (P == 0 || delta), "add_rmsnorm_ext: bad sizes T=%d H=%d P=%d", T, H, P);
  IB_CHECK_ARG(!mix || (state && seg_slot), "add_rmsnorm_ext: the shift needs the state and the rows' slots");
  const size_t smem = (size_t)H * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "add_rmsnorm_ext: hidden size %d needs %zu bytes of shared memory, more than 200 KiB", H, smem);
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, T, row_threads(H), smem, stream, x, delta, P, (size_t)delta_stride, bias, w, eps, mix, state, (size_t)slot_stride, seg_slot, o, H);
  };
  if (out_dtype == IB_F32) {
    if (mix) go(add_rmsnorm_ext_kernel<float, true>, (float*)out);
    else go(add_rmsnorm_ext_kernel<float, false>, (float*)out);
  } else if (out_dtype == IB_BF16) {
    if (mix) go(add_rmsnorm_ext_kernel<__nv_bfloat16, true>, (__nv_bfloat16*)out);
    else go(add_rmsnorm_ext_kernel<__nv_bfloat16, false>, (__nv_bfloat16*)out);
  } else {
    return ib_set_error("add_rmsnorm_ext: unknown output dtype %d", out_dtype);
  }
  IB_CHECK_LAUNCH("add_rmsnorm_ext");
  return 0;
}

extern "C" int ib_loop_pack(float* x, const float* delta, int P, long long delta_stride, const float* x0, const float* step, void* packed, int act_dtype, int T, int H,
                            cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && P >= 0 && (P == 0 || delta), "loop_pack: bad sizes T=%d H=%d P=%d", T, H, P);
  const dim3 grid((unsigned)T, (unsigned)min((H + 255) / 256, 64));
  if (act_dtype == IB_F32) ib::launch(loop_pack_kernel<float>, grid, 256, 0, stream, x, delta, P, (size_t)delta_stride, x0, step, (float*)packed, H);
  else if (act_dtype == IB_BF16) ib::launch(loop_pack_kernel<__nv_bfloat16>, grid, 256, 0, stream, x, delta, P, (size_t)delta_stride, x0, step, (__nv_bfloat16*)packed, H);
  else return ib_set_error("loop_pack: unknown activation dtype %d", act_dtype);
  IB_CHECK_LAUNCH("loop_pack");
  return 0;
}

extern "C" int ib_add_bias_rows(float* v, const float* bias, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0, "add_bias_rows: bad sizes T=%d H=%d", T, H);
  ib::launch(add_bias_rows_kernel, dim3((unsigned)T, (unsigned)min((H + 255) / 256, 64)), 256, 0, stream, v, bias, H);
  IB_CHECK_LAUNCH("add_bias_rows");
  return 0;
}

extern "C" int ib_xielu_rows(const float* z, int P, long long stride, const float* pq, void* act, int act_dtype, int T, int I, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && I > 0 && P >= 1 && T <= 65535, "xielu_rows: bad sizes T=%d I=%d P=%d", T, I, P);
  dim3 grid((unsigned)min((I + 255) / 256, 64), (unsigned)T);
  if (act_dtype == IB_F32) ib::launch(xielu_rows_kernel<float>, grid, 256, 0, stream, z, P, (size_t)stride, pq, (float*)act, I);
  else if (act_dtype == IB_BF16) ib::launch(xielu_rows_kernel<__nv_bfloat16>, grid, 256, 0, stream, z, P, (size_t)stride, pq, (__nv_bfloat16*)act, I);
  else return ib_set_error("xielu_rows: unknown output dtype %d", act_dtype);
  IB_CHECK_LAUNCH("xielu_rows");
  return 0;
}

extern "C" int ib_gated_rmsnorm(const float* o, const float* w, float eps, const float* gate, int P, long long gate_stride, int gate_row, float scale, void* out,
                                int out_dtype, int out_row, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && P >= 1 && out_row >= H && gate_row >= H, "gated_rmsnorm: bad sizes T=%d H=%d P=%d", T, H, P);
  if (out_dtype == IB_F32) ib::launch(gated_rmsnorm_kernel<float>, T, row_threads(H), 0, stream, o, w, eps, gate, P, (size_t)gate_stride, gate_row, scale, (float*)out, out_row, H);
  else if (out_dtype == IB_BF16)
    ib::launch(gated_rmsnorm_kernel<__nv_bfloat16>, T, row_threads(H), 0, stream, o, w, eps, gate, P, (size_t)gate_stride, gate_row, scale, (__nv_bfloat16*)out, out_row, H);
  else return ib_set_error("gated_rmsnorm: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}
