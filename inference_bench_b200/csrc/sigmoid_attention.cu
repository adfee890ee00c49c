// Attention whose weights are sigmoids, behind a short convolution of its projections.
//
// Per token t of a request, with u_t = [q | k | v] the biased projections of the layer's input (float32 partial sums, added in order):
//     y_t[c] = sum_j w[j][c] u_(t - taps + 1 + j)[c]                  a causal convolution over time on every channel, zeros before the start
//     q = y_q * (1 + coef * ln(floor((p + 1) / every) + 1))           a temperature that grows with the position p
//     v = y_v / sqrt(mean(y_v^2) + eps) per head                      (cached so);   k = y_k
//     s_ij = (q_i . k_j) * scale - r1_h * ln(1 + r2_h * (i - j)) + pb_h   for every j <= i;     o_i = sum_j sigmoid(s_ij) v_j
// The weights are not normalised over the keys, so partial sums over slices of the keys simply add. The last taps - 1 rows of u are state
// of the request (a fixed-size slot). Everything between the projection's sums and the cache is float32.
//
//  * qkv_conv: a warp per (token, head of q, k or v): convolution (rows before the segment's first token come from the request's state),
//    temperature, value norm; writes q in the activation dtype and k, v into the paged cache. It only reads the state.
//  * conv_state_shift: the request's state becomes the last taps - 1 rows of u (old rows move up when the step brought fewer); it runs
//    after every reader of the old state.
//  * sigmoid_attention: any sizes, float32 or bfloat16 storage with float32 arithmetic: a warp per (token, head, slice of the keys), a lane
//    per key for the scores and per output column for the sum. With slices the partial sums go to scratch and sigmoid_combine adds them
//    in the order of the slices.
//  * sigmoid_attention_mma: bfloat16, head sizes that are multiples of 16, on the tensor cores (m16n8k16): a CTA of four warps owns 16
//    query rows of one (request, kv head): the group's heads of one token, or of consecutive tokens of a prompt portion, and walks
//    the keys in tiles of 64 through shared memory (cp.async, two buffers). Warp w computes S for keys 16w..16w+15, applies the distance bias and
//    the sigmoid in float32, rounds the weights to bfloat16 as the operand of the second product, and the warps then split the value
//    columns of O += P V. That form serves decoded tokens (whose keys may also be cut into slices) and head sizes above 128; prompt portions
//    of head sizes up to 128 run sigmoid_prefill_mma, where a warp owns sixteen of the CTA's 64 rows over all of a tile's keys and the
//    weights stay in registers between the two products.
#include <type_traits>

#include "kv_view.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename A, typename C>
__global__ void qkv_conv_kernel(const float* __restrict__ proj, int P, size_t stride_p, int R, const float* __restrict__ bias, const float* __restrict__ conv_w,
                                int taps, float* conv_state, size_t slot_stride, const int* __restrict__ seg_of_token,
                                const int* __restrict__ seg_start, const int* __restrict__ seg_slot, const int* __restrict__ positions, int T, int heads,
                                int qk_dim, int v_dim, float temp_coef, int temp_every, int v_norm, float eps, A* __restrict__ q_out, IbKvView kv,
                                unsigned* __restrict__ status, int shift_state) {
  // shift_state: every segment of the step is a single token, so the warp that reads a request's state rows of its channels is their only reader
  // and moves them up itself (the new last row is this token's u); otherwise conv_state_shift does that after this kernel.
  // proj: [P][T][R], R = (heads + kv_heads) * qk_dim + kv_heads * v_dim; bias: [R] or null; conv_w: [taps][R] (the last row is the current
  // token's) or null for no convolution; conv_state: [slots][taps - 1][R] (rows of u, biased). temp_every <= 0: no temperature.
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int kvh = kv.kv_heads, slots = heads + 2 * kvh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * slots) return;
  const int t = (int)(item / slots), j = (int)(item % slots);
  const bool is_q = j < heads, is_k = !is_q && j < heads + kvh;
  const int hd = (is_q || is_k) ? qk_dim : v_dim;
  const int col0 = (is_q || is_k) ? j * qk_dim : (heads + kvh) * qk_dim + (j - heads - kvh) * v_dim;
  const int s = seg_of_token[t], t0 = seg_start[s];
  float* old = conv_state ? conv_state + (size_t)seg_slot[s] * slot_stride : nullptr;
  float y[kMaxHeadDim / 32];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) {
    const int d = lane + 32 * r;
    y[r] = 0.f;
    if (d >= hd) continue;
    const int c = col0 + d;
    auto u_at = [&](int row) {
      if (row < t0) return old[(size_t)((taps - 1) + (row - t0)) * R + c];
      const float* src = proj + (size_t)row * R + c;
      float v = src[0];
#pragma unroll 4
      for (int p = 1; p < P; p++) v += src[p * stride_p];
      return bias ? v + bias[c] : v;
    };
    float acc;
    if (conv_w) {
      acc = 0.f;
      for (int k = 0; k < taps; k++) acc = __fmaf_rn(conv_w[(size_t)k * R + c], u_at(t - (taps - 1) + k), acc);
      if (shift_state && taps > 1) {
        for (int k = 0; k + 2 < taps; k++) old[(size_t)k * R + c] = old[(size_t)(k + 1) * R + c];
        old[(size_t)(taps - 2) * R + c] = u_at(t);
      }
    } else {
      acc = u_at(t);
    }
    y[r] = acc;
    ss = __fmaf_rn(acc, acc, ss);
  }
  float f = 1.f;
  if (is_q && temp_every > 0) f = 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
  if (!is_q && !is_k && v_norm) f = 1.f / sqrtf(ib::warp_sum(ss) / (float)hd + eps);
  if (is_q) {
    A* dst = q_out + ((size_t)t * heads + j) * hd;
#pragma unroll
    for (int r = 0; r < kMaxHeadDim / 32; r++) {
      const int d = lane + 32 * r;
      if (d < hd) dst[d] = ib::from_f32<A>(y[r] * f);
    }
    return;
  }
  const int head = is_k ? j - heads : j - heads - kvh;
  const long long off = ib::kv_offset(kv, s, positions[t], head);
  if (off < 0) {
    if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
    return;
  }
  C* dst = (C*)kv.base + off + (is_k ? 0 : kv.v_offset);
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) {
    const int d = lane + 32 * r;
    if (d < hd) dst[d] = ib::from_f32<C>(y[r] * f);
  }
}

// Row r of a request's state becomes u at the segment's row n_seg - (taps - 1) + r, or the old row n_seg + r when that lies before the
// segment. Row r is written after row r + n_seg was read and later rows read only rows further on: in place, in rising order.
__global__ void conv_state_shift_kernel(const float* __restrict__ proj, int P, size_t stride_p, int R, const float* __restrict__ bias, int taps,
                                        float* __restrict__ conv_state, size_t slot_stride, const int* __restrict__ seg_start, const int* __restrict__ seg_slot) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= R) return;
  const int t0 = seg_start[s], n_seg = seg_start[s + 1] - t0;
  float* cs = conv_state + (size_t)seg_slot[s] * slot_stride;
  for (int r = 0; r < taps - 1; r++) {
    const int rel = n_seg - (taps - 1) + r;
    float v;
    if (rel >= 0) {
      const float* src = proj + (size_t)(t0 + rel) * R + c;
      v = src[0];
      for (int p = 1; p < P; p++) v += src[p * stride_p];
      if (bias) v += bias[c];
    } else {
      v = cs[(size_t)(n_seg + r) * R + c];
    }
    cs[(size_t)r * R + c] = v;
  }
}

// lane owns output columns lane, lane + 32, ...
template <typename A, typename C>
__global__ void sigmoid_attention_kernel(const A* __restrict__ q, IbKvView kv, const int* __restrict__ positions, const int* __restrict__ seg_of_token, float scale,
                                         const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb, A* __restrict__ out,
                                         float* __restrict__ part, int T, int heads, int qk_dim, int v_dim, int n_slices, int slice_keys,
                                         unsigned* __restrict__ status) {
  __shared__ float qs[kWarps][kMaxHeadDim];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads), slice = blockIdx.y;
  const int kvhead = h / (heads / kv.kv_heads);
  const int pos = positions[t], seg = seg_of_token[t];
  const int lo = slice * slice_keys, hi = min(pos, lo + slice_keys - 1);
  const A* qrow = q + ((size_t)t * heads + h) * qk_dim;
  for (int d = lane; d < qk_dim; d += 32) qs[warp][d] = ib::to_f32<A>(qrow[d]);
  __syncwarp();
  const float a1 = r1 ? r1[h] : 0.f, a2 = r2 ? r2[h] : 0.f, b0 = pb ? pb[h] : 0.f;
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) acc[r] = 0.f;
  const C* base = (const C*)kv.base;
  for (int k0 = lo; k0 <= hi; k0 += 32) {
    const int key = k0 + lane;
    long long off = -1;
    float p = 0.f;
    if (key <= hi) {
      off = ib::kv_offset(kv, seg, key, kvhead);
      if (off < 0) {
        atomicOr(status, IB_ERR_BAD_PAGE);
      } else {
        const C* kr = base + off;
        float dot = 0.f;
        for (int d = 0; d < qk_dim; d++) dot = __fmaf_rn(qs[warp][d], ib::to_f32<C>(kr[d]), dot);
        const float sc = dot * scale - a1 * log1pf(a2 * (float)(pos - key)) + b0;
        p = 1.f / (1.f + expf(-sc));
      }
    }
    const int n = min(32, hi - k0 + 1);
    for (int jj = 0; jj < n; jj++) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long oj = __shfl_sync(0xffffffffu, off, jj);
      if (oj < 0) continue;
      const C* vr = base + oj + kv.v_offset;
#pragma unroll
      for (int r = 0; r < kMaxHeadDim / 32; r++) {
        const int d = lane + 32 * r;
        if (d < v_dim) acc[r] = __fmaf_rn(pj, ib::to_f32<C>(vr[d]), acc[r]);
      }
    }
  }
  if (n_slices == 1) {
    A* orow = out + ((size_t)t * heads + h) * v_dim;
#pragma unroll
    for (int r = 0; r < kMaxHeadDim / 32; r++) {
      const int d = lane + 32 * r;
      if (d < v_dim) orow[d] = ib::from_f32<A>(acc[r]);
    }
    return;
  }
  float* po = part + (((size_t)t * heads + h) * n_slices + slice) * v_dim;
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) {
    const int d = lane + 32 * r;
    if (d < v_dim) po[d] = acc[r];
  }
}

// out[row] = sum over the slices of (token, head) `row`'s partial sums, in the order of the slices.
// With positions, a token's slices end with the one that holds its own position (later ones were never written).
template <typename O>
__global__ void sigmoid_combine_kernel(const float* __restrict__ part, O* __restrict__ out, int v_dim, int n_slices, const int* __restrict__ positions, int heads,
                                       int slice_keys) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const float* src = part + (size_t)blockIdx.x * n_slices * v_dim;
  const int n = positions ? min(n_slices, positions[blockIdx.x / heads] / slice_keys + 1) : n_slices;
  for (int d = threadIdx.x; d < v_dim; d += blockDim.x) {
    float a = src[d];
    for (int s = 1; s < n; s++) a += src[(size_t)s * v_dim + d];
    out[(size_t)blockIdx.x * v_dim + d] = ib::from_f32<O>(a);
  }
}

// ---------------------------------------------------------------- tensor cores
constexpr int kKeys = 64;     // keys of a tile
constexpr int kMmaWarps = 4;  // each takes 16 of a tile's keys for S, and a share of the value columns for O

// The CTA's R = 16 MT query rows: row r is head r % group of the kv head's group, of token tok0 + r / group (group = query heads a kv head, at most 16).
// A prompt portion fills 64 rows (every key and value tile is then read once for 64 / group tokens); a decoded token has its group's rows alone.
// NV: 16-column chunks of the output a warp owns at most.
template <int NV, int MT>
__global__ void __launch_bounds__(kMmaWarps * 32) sigmoid_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                                                               const int* __restrict__ seg_of_token, const int2* __restrict__ units, float scale,
                                                                               const float* __restrict__ r1, const float* __restrict__ r2,
                                                                               const float* __restrict__ pb, __nv_bfloat16* __restrict__ out,
                                                                               float* __restrict__ part, int heads, int qk_dim, int v_dim, int n_slices,
                                                                               int slice_keys, unsigned* __restrict__ status) {
  constexpr int R = 16 * MT;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float4 s_row[R];                                 // per row: position (as bits; -1: no such row), r1, r2, pb of its head
  const int qb = (qk_dim + 63) / 64, vb = (v_dim + 63) / 64;
  const uint32_t k_bytes = (uint32_t)qb * kKeys * 128, v_bytes = (uint32_t)vb * kKeys * 128;
  const uint32_t s_k = mt::smem_u32(smem);                    // two key tiles
  const uint32_t s_v = s_k + 2 * k_bytes;                     // two value tiles
  const uint32_t s_q = s_v + 2 * v_bytes;                     // [R][qk_dim]
  const uint32_t s_p = s_q + (uint32_t)qb * R * 128;          // [R][64]
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int group = heads / kv.kv_heads;
  const int per = R / group;                                   // tokens a CTA holds at most
  const int kvhead = blockIdx.x;
  const int ui = gridDim.y - 1 - blockIdx.y;                   // the last units first: in a prompt portion they see the most keys
  int tok0 = ui, ntok = 1;
  if (units) {
    const int2 u = units[ui];
    tok0 = u.x, ntok = u.y;
  }
  ntok = min(ntok, per);
  const int slice = blockIdx.z;
  const int seg = seg_of_token[tok0];
  const int last_pos = positions[tok0 + ntok - 1];
  const int lo = slice * slice_keys, hi = min(last_pos, lo + slice_keys - 1);
  for (int r = tid; r < R; r += kMmaWarps * 32) {
    const int tl = r / group, h = kvhead * group + (r - tl * group);
    const int pos = tl < ntok ? positions[tok0 + tl] : -1;
    s_row[r] = make_float4(__int_as_float(pos), r1 ? r1[h] : 0.f, r2 ? r2[h] : 0.f, pb ? pb[h] : 0.f);
  }
  // queries, swizzled [R][qk_dim]
  for (int idx = tid; idx < R * (qk_dim / 8); idx += kMmaWarps * 32) {
    const int r = idx / (qk_dim / 8), c = idx - r * (qk_dim / 8);
    const int tl = r / group, hh = r - tl * group;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (tl < ntok) w = *(const uint4*)(q + ((size_t)(tok0 + tl) * heads + kvhead * group + hh) * qk_dim + c * 8);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(s_q + mt::tile_offset<64, R>(r, c)), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
  }
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
  // a thread copies the 16-byte pieces tid % 8, + 8, ... of rows tid / 8 + 16 i of the tile, keys and values
  auto issue_tile = [&](int k0, int buf) {
#pragma unroll
    for (int i = 0; i < kKeys / 16; i++) {
      const int row = (tid >> 3) + 16 * i, key = k0 + row;
      long long off = -1;
      if (key <= hi) {
        off = ib::kv_offset(kv, seg, key, kvhead);
        if (off < 0) atomicOr(status, IB_ERR_BAD_PAGE);
      }
      for (int c = tid & 7; c < qk_dim / 8; c += 8) {
        const uint32_t at = s_k + buf * k_bytes + mt::tile_offset<64, kKeys>(row, c);
        if (off >= 0) mt::cp_async16(at, base + off + c * 8);
        else mt::st_shared_zero16(at);
      }
      for (int c = tid & 7; c < v_dim / 8; c += 8) {
        const uint32_t at = s_v + buf * v_bytes + mt::tile_offset<64, kKeys>(row, c);
        if (off >= 0) mt::cp_async16(at, base + off + kv.v_offset + c * 8);
        else mt::st_shared_zero16(at);
      }
    }
    mt::cp_async_commit();
  };
  float o[MT][NV][2][4];
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int i = 0; i < NV; i++)
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[a][i][n][e] = 0.f;
  const int n_tiles = hi >= lo ? (hi - lo) / kKeys + 1 : 0;
  const int n_vc = v_dim / 16;                                 // 16-column chunks of the output; warp w owns chunks w, w + 4, ...
  if (n_tiles > 0) issue_tile(lo, 0);
  for (int j = 0; j < n_tiles; j++) {
    const int k0 = lo + j * kKeys, buf = j & 1;
    mt::cp_async_wait<0>();
    __syncthreads();                                           // tile j is here; everybody is done with tile j - 1 and with P (and s_row is written)
    if (j + 1 < n_tiles) issue_tile(k0 + kKeys, buf ^ 1);
    const uint32_t kt = s_k + buf * k_bytes, vt = s_v + buf * v_bytes;
    // ---- S: this warp's 16 keys, every row tile
    float s[MT][2][4];
#pragma unroll
    for (int a = 0; a < MT; a++)
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) s[a][n][e] = 0.f;
    for (int kk = 0; kk < qk_dim / 16; kk++) {
      uint32_t fb[4];
      mt::load_k_frag<64, kKeys>(kt, 16 * warp, kk, lane, fb);
#pragma unroll
      for (int a = 0; a < MT; a++) {
        uint32_t fa[4];
        mt::load_a_frag<64, R>(s_q, 16 * a, kk, lane, fa);
        mt::mma_16816(s[a][0], fa, fb[0], fb[1]);
        mt::mma_16816(s[a][1], fa, fb[2], fb[3]);
      }
    }
    // ---- weights: float32 bias and sigmoid, bfloat16 as the operand of the second product
#pragma unroll
    for (int a = 0; a < MT; a++) {
      const float4 ra = s_row[16 * a + g], rb = s_row[16 * a + g + 8];
      const int pa = __float_as_int(ra.x), pbs = __float_as_int(rb.x);
#pragma unroll
      for (int n = 0; n < 2; n++) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int key = k0 + 16 * warp + 8 * n + 2 * t4 + (e & 1);
          const bool second = e >> 1;
          const int rp = second ? pbs : pa;
          float w = 0.f;
          if (key <= hi && key <= rp) {
            const float c1 = second ? rb.y : ra.y, c2 = second ? rb.z : ra.z, c0 = second ? rb.w : ra.w;
            const float sc = s[a][n][e] * scale - c1 * __logf(1.f + c2 * (float)(rp - key)) + c0;
            w = __fdividef(1.f, 1.f + __expf(-sc));
          }
          p[e] = w;
        }
        const int chunk = 2 * warp + n;                        // this warp's 16 keys are chunks 2 warp, 2 warp + 1 of the P tile's 64
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_p + mt::tile_offset<64, R>(16 * a + g, chunk) + 4 * t4), "r"(mt::pack_bf16(p[0], p[1])) : "memory");
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_p + mt::tile_offset<64, R>(16 * a + g + 8, chunk) + 4 * t4), "r"(mt::pack_bf16(p[2], p[3])) : "memory");
      }
    }
    __syncthreads();
    // ---- O += P V: this warp's column chunks, every row tile
#pragma unroll
    for (int ks = 0; ks < kKeys / 16; ks++) {
      uint32_t fa[MT][4];
#pragma unroll
      for (int a = 0; a < MT; a++) mt::load_a_frag<64, R>(s_p, 16 * a, ks, lane, fa[a]);
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int dp = warp + kMmaWarps * i;                   // the 16-column chunk
        if (dp >= n_vc) continue;
        uint32_t fv[4];
        mt::load_v_frag<64, kKeys>(vt, 16 * ks, dp, lane, fv);
#pragma unroll
        for (int a = 0; a < MT; a++) {
          mt::mma_16816(o[a][i][0], fa[a], fv[0], fv[1]);
          mt::mma_16816(o[a][i][1], fa[a], fv[2], fv[3]);
        }
      }
    }
  }
  // ---- out
  __syncthreads();   // (a CTA without tiles has not yet met a barrier after writing s_row)
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      const int r = 16 * a + g + 8 * rr, tl = r / group;
      if (tl >= ntok) continue;
      const size_t th = (size_t)(tok0 + tl) * heads + kvhead * group + (r - tl * group);
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int dp = warp + kMmaWarps * i;
        if (dp >= n_vc) continue;
#pragma unroll
        for (int n = 0; n < 2; n++) {
          if (n_slices == 1) *(uint32_t*)(out + th * v_dim + dp * 16 + 8 * n + 2 * t4) = mt::pack_bf16(o[a][i][n][2 * rr], o[a][i][n][2 * rr + 1]);
          else *(float2*)(part + (th * n_slices + slice) * v_dim + dp * 16 + 8 * n + 2 * t4) = make_float2(o[a][i][n][2 * rr], o[a][i][n][2 * rr + 1]);
        }
      }
    }
}

// Prompt portions: 64 query rows a CTA, sixteen a warp (row r is head r % group of token tok0 + r / group). A warp keeps its rows' query
// fragments, its scores and its output in registers and walks every key tile on its own: S = Q K^T for all 64 keys, the bias and the sigmoid in
// float32, the weights repacked from the accumulators' layout into the first operand of O += P V without a trip through shared memory. The warps
// meet only where a key and value tile is handed over (one barrier a tile); a warp skips a tile none of its rows sees.
// NQ, NVC: 16-value steps of a key row and 16-column chunks of a value row at most (head sizes up to 16 NQ and 16 NVC).
template <int NQ, int NVC>
__global__ void __launch_bounds__(kMmaWarps * 32) sigmoid_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                                                             const int* __restrict__ seg_of_token, const int2* __restrict__ units, float scale,
                                                                             const float* __restrict__ r1, const float* __restrict__ r2,
                                                                             const float* __restrict__ pb, __nv_bfloat16* __restrict__ out,
                                                                             float* __restrict__ part, int heads, int qk_dim, int v_dim, int n_slices,
                                                                             int slice_keys, unsigned* __restrict__ status) {
  // n_slices > 1: blockIdx.z is a slice of slice_keys keys; a CTA whose tokens all lie before its slice leaves, and a row's partial sums go to
  // part[(token, head)][slice] only where the row's position reaches the slice (sigmoid_combine adds those).
  constexpr int R = 16 * kMmaWarps;
  extern __shared__ __align__(128) unsigned char smem[];
  const int qb = (qk_dim + 63) / 64, vb = (v_dim + 63) / 64;
  const uint32_t k_bytes = (uint32_t)qb * kKeys * 128, v_bytes = (uint32_t)vb * kKeys * 128;
  const uint32_t s_k = mt::smem_u32(smem);                    // two key tiles
  const uint32_t s_v = s_k + 2 * k_bytes;                     // two value tiles
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int group = heads / kv.kv_heads;
  const int per = R / group;
  const int kvhead = blockIdx.x;
  const int ui = gridDim.y - 1 - blockIdx.y;                   // the last units first: they see the most keys
  const int2 u = units[ui];
  const int tok0 = u.x, ntok = min(u.y, per);
  const int seg = seg_of_token[tok0];
  const int slice = blockIdx.z, lo = slice * slice_keys;
  const int hi = min(positions[tok0 + ntok - 1], lo + slice_keys - 1);
  if (hi < lo) return;
  // the two rows this thread sees in its accumulators
  int rpos[2], rtok[2], rhead[2];
  float c1[2], c2[2], c0[2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = 16 * warp + g + 8 * e, tl = r / group;
    rhead[e] = kvhead * group + (r - tl * group);
    rtok[e] = tl < ntok ? tok0 + tl : -1;
    rpos[e] = tl < ntok ? positions[tok0 + tl] : -1;
    c1[e] = r1 ? r1[rhead[e]] : 0.f, c2[e] = r2 ? r2[rhead[e]] : 0.f, c0[e] = pb ? pb[rhead[e]] : 0.f;
  }
  // the last position any row of this warp holds: tiles beyond it are not for this warp; the first: tiles that end before it need no mask
  int warp_hi = max(rpos[0], rpos[1]), warp_lo = min(rpos[0], rpos[1]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    warp_hi = max(warp_hi, __shfl_xor_sync(0xffffffffu, warp_hi, o));
    warp_lo = min(warp_lo, __shfl_xor_sync(0xffffffffu, warp_lo, o));
  }
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
  auto issue_tile = [&](int k0, int buf) {
#pragma unroll
    for (int i = 0; i < kKeys / 16; i++) {
      const int row = (tid >> 3) + 16 * i, key = k0 + row;
      long long off = -1;
      if (key <= hi) {
        off = ib::kv_offset(kv, seg, key, kvhead);
        if (off < 0) atomicOr(status, IB_ERR_BAD_PAGE);
      }
      for (int c = tid & 7; c < qk_dim / 8; c += 8) {
        const uint32_t at = s_k + buf * k_bytes + mt::tile_offset<64, kKeys>(row, c);
        if (off >= 0) mt::cp_async16(at, base + off + c * 8);
        else mt::st_shared_zero16(at);
      }
      for (int c = tid & 7; c < v_dim / 8; c += 8) {
        const uint32_t at = s_v + buf * v_bytes + mt::tile_offset<64, kKeys>(row, c);
        if (off >= 0) mt::cp_async16(at, base + off + kv.v_offset + c * 8);
        else mt::st_shared_zero16(at);
      }
    }
    mt::cp_async_commit();
  };
  const int nq = qk_dim / 16, n_vc = v_dim / 16;
  const int n_tiles = (hi - lo) / kKeys + 1;
  issue_tile(lo, 0);
  // the query fragments straight from memory, once: (row g, values 2 t4..) (row g + 8, the same) (row g, values 8 + 2 t4..) (row g + 8, the same) of every 16-value step
  uint32_t qf[NQ][4];
  {
    const __nv_bfloat16* q0 = rtok[0] >= 0 ? q + ((size_t)rtok[0] * heads + rhead[0]) * qk_dim + 2 * t4 : nullptr;
    const __nv_bfloat16* q1 = rtok[1] >= 0 ? q + ((size_t)rtok[1] * heads + rhead[1]) * qk_dim + 2 * t4 : nullptr;
#pragma unroll
    for (int kk = 0; kk < NQ; kk++) {
      qf[kk][0] = qf[kk][1] = qf[kk][2] = qf[kk][3] = 0u;
      if (kk >= nq) continue;
      if (q0) qf[kk][0] = *(const uint32_t*)(q0 + 16 * kk), qf[kk][2] = *(const uint32_t*)(q0 + 16 * kk + 8);
      if (q1) qf[kk][1] = *(const uint32_t*)(q1 + 16 * kk), qf[kk][3] = *(const uint32_t*)(q1 + 16 * kk + 8);
    }
  }
  float o[NVC][2][4];
#pragma unroll
  for (int i = 0; i < NVC; i++)
#pragma unroll
    for (int n = 0; n < 2; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[i][n][e] = 0.f;
  for (int j = 0; j < n_tiles; j++) {
    const int k0 = lo + j * kKeys, buf = j & 1;
    mt::cp_async_wait<0>();
    __syncthreads();                                           // tile j is here; everybody is done with tile j - 1
    if (j + 1 < n_tiles) issue_tile(k0 + kKeys, buf ^ 1);
    if (k0 > warp_hi) continue;
    const uint32_t kt = s_k + buf * k_bytes, vt = s_v + buf * v_bytes;
    float sc[kKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kKeys / 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) sc[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < NQ; kk++) {
      if (kk >= nq) continue;
#pragma unroll
      for (int n2 = 0; n2 < kKeys / 16; n2++) {
        uint32_t fb[4];
        mt::load_k_frag<64, kKeys>(kt, 16 * n2, kk, lane, fb);
        mt::mma_16816(sc[2 * n2], qf[kk], fb[0], fb[1]);
        mt::mma_16816(sc[2 * n2 + 1], qf[kk], fb[2], fb[3]);
      }
    }
    uint32_t pa[kKeys / 16][4];
    const bool all_seen = k0 + kKeys - 1 <= min(warp_lo, hi);   // every key of the tile is seen by every row of the warp
    const float d0[2] = {(float)(rpos[0] - k0 - 2 * t4), (float)(rpos[1] - k0 - 2 * t4)};   // distance to the thread's first key of the tile
#pragma unroll
    for (int n = 0; n < kKeys / 8; n++) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int rr = e >> 1;
        const float dist = d0[rr] - (float)(8 * n + (e & 1));
        const float v = sc[n][e] * scale - c1[rr] * __logf(__fmaf_rn(c2[rr], dist, 1.f)) + c0[rr];
        float w = __fdividef(1.f, 1.f + __expf(-v));
        if (!all_seen && (dist < 0.f || k0 + 8 * n + 2 * t4 + (e & 1) > hi)) w = 0.f;
        p[e] = w;
      }
      // the accumulators of two neighbouring 8-key tiles are the first operand's fragment of one 16-key step
      pa[n >> 1][2 * (n & 1)] = mt::pack_bf16(p[0], p[1]);
      pa[n >> 1][2 * (n & 1) + 1] = mt::pack_bf16(p[2], p[3]);
    }
#pragma unroll
    for (int ks = 0; ks < kKeys / 16; ks++) {
#pragma unroll
      for (int dp = 0; dp < NVC; dp++) {
        if (dp >= n_vc) continue;
        uint32_t fv[4];
        mt::load_v_frag<64, kKeys>(vt, 16 * ks, dp, lane, fv);
        mt::mma_16816(o[dp][0], pa[ks], fv[0], fv[1]);
        mt::mma_16816(o[dp][1], pa[ks], fv[2], fv[3]);
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; rr++) {
    if (rtok[rr] < 0 || rpos[rr] < lo) continue;
    const size_t th = (size_t)rtok[rr] * heads + rhead[rr];
#pragma unroll
    for (int dp = 0; dp < NVC; dp++) {
      if (dp >= n_vc) continue;
#pragma unroll
      for (int n = 0; n < 2; n++) {
        if (n_slices == 1) *(uint32_t*)(out + th * v_dim + dp * 16 + 8 * n + 2 * t4) = mt::pack_bf16(o[dp][n][2 * rr], o[dp][n][2 * rr + 1]);
        else *(float2*)(part + (th * n_slices + slice) * v_dim + dp * 16 + 8 * n + 2 * t4) = make_float2(o[dp][n][2 * rr], o[dp][n][2 * rr + 1]);
      }
    }
  }
}

size_t sigmoid_mma_smem(int qk_dim, int v_dim, int rows) {
  const int qb = (qk_dim + 63) / 64, vb = (v_dim + 63) / 64;
  return (size_t)2 * (qb + vb) * kKeys * 128 + (size_t)qb * rows * 128 + (size_t)rows * 128;
}

int check_view(const char* name, const IbKvView* kv, int heads, int qk_dim, int v_dim) {
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "%s: the cache view has a null pointer", name);
  IB_CHECK_ARG(kv->kv_heads > 0 && heads > 0 && heads % kv->kv_heads == 0, "%s: %d query heads are not a multiple of %d kv heads", name, heads, kv->kv_heads);
  IB_CHECK_ARG(qk_dim > 0 && v_dim > 0 && qk_dim <= kv->head_dim && v_dim <= kv->head_dim && kv->head_dim <= kMaxHeadDim,
               "%s: head sizes %d and %d must be positive and fit the cache's row of %d (at most %d)", name, qk_dim, v_dim, kv->head_dim, kMaxHeadDim);
  IB_CHECK_ARG(kv->page_size > 0 && kv->num_pages > 0 && kv->table_stride > 0, "%s: bad page geometry", name);
  IB_CHECK_ARG(kv->dtype == IB_F32 || kv->dtype == IB_BF16, "%s: unknown cache dtype %d", name, kv->dtype);
  return 0;
}

}  // namespace

extern "C" int ib_qkv_conv(const float* proj, int P, long long stride_p, const float* bias, const float* conv_w, int taps, float* conv_state, long long slot_stride,
                           const int* seg_of_token, const int* seg_start, const int* seg_slot, int n_segments, const int* positions, int T, int heads, int qk_dim,
                           int v_dim, float temp_coef, int temp_every, int v_norm, float eps, void* q_out, int act_dtype, const IbKvView* kv, unsigned* status,
                           int single_tokens, cudaStream_t stream) {
  // single_tokens: every segment brings one token (n_segments == T): the state is moved up inside the one kernel.
  // conv_w null (taps 1 without weights): the projections go through as they are. conv_state may be null when taps == 1.
  if (T == 0) return 0;
  if (check_view("qkv_conv", kv, heads, qk_dim, v_dim)) return 1;
  IB_CHECK_ARG(P >= 1 && taps >= 1 && (taps == 1 || (conv_w && conv_state)), "qkv_conv: bad sizes P=%d taps=%d", P, taps);
  IB_CHECK_ARG(!single_tokens || n_segments == T, "qkv_conv: %d segments of single tokens do not make %d tokens", n_segments, T);
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "qkv_conv: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  const int R = (heads + kv->kv_heads) * qk_dim + kv->kv_heads * v_dim;
  const long long items = (long long)T * (heads + 2 * kv->kv_heads);
  const unsigned blocks = (unsigned)((items + kWarps - 1) / kWarps);
  auto go = [&](auto kernel, auto* qo) {
    ib::launch(kernel, blocks, kWarps * 32, 0, stream, proj, P, (size_t)stride_p, R, bias, conv_w, taps, conv_state, (size_t)slot_stride, seg_of_token,
               seg_start, seg_slot, positions, T, heads, qk_dim, v_dim, temp_coef, temp_every, v_norm, eps, qo, *kv, status, single_tokens);
  };
  if (act_dtype == IB_F32) go(qkv_conv_kernel<float, float>, (float*)q_out);
  else go(qkv_conv_kernel<__nv_bfloat16, __nv_bfloat16>, (__nv_bfloat16*)q_out);
  IB_CHECK_LAUNCH("qkv_conv");
  if (taps > 1 && !single_tokens) {
    IB_CHECK_ARG(n_segments > 0 && n_segments <= 65535 * 32, "qkv_conv: %d segments", n_segments);
    ib::launch(conv_state_shift_kernel, dim3((unsigned)n_segments, (unsigned)((R + 127) / 128)), 128, 0, stream, proj, P, (size_t)stride_p, R, bias, taps, conv_state,
               (size_t)slot_stride, seg_start, seg_slot);
    IB_CHECK_LAUNCH("conv_state_shift");
  }
  return 0;
}

extern "C" int ib_sigmoid_combine(const float* part, void* out, int out_dtype, int rows, int v_dim, int n_slices, const int* positions, int heads, int slice_keys,
                                  cudaStream_t stream) {
  // positions: null (every slice of every row was written) or the tokens' positions (row = token * heads + head; slices beyond a token's own were not written).
  if (rows == 0) return 0;
  if (out_dtype == IB_F32) ib::launch(sigmoid_combine_kernel<float>, (unsigned)rows, 128, 0, stream, part, (float*)out, v_dim, n_slices, positions, heads, slice_keys);
  else if (out_dtype == IB_BF16)
    ib::launch(sigmoid_combine_kernel<__nv_bfloat16>, (unsigned)rows, 128, 0, stream, part, (__nv_bfloat16*)out, v_dim, n_slices, positions, heads, slice_keys);
  else return ib_set_error("sigmoid_combine: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("sigmoid_combine");
  return 0;
}

extern "C" int ib_sigmoid_attention(const void* q, int act_dtype, const IbKvView* kv, const int* positions, const int* seg_of_token, float scale, const float* r1,
                                    const float* r2, const float* pb, void* out, float* part, int T, int heads, int qk_dim, int v_dim, int n_slices, int slice_keys,
                                    unsigned* status, cudaStream_t stream) {
  // r1, r2: the distance bias r1[h] * ln(1 + r2[h] * distance) taken off the score (null: none); pb: a number per head added to it (null: none).
  if (T == 0) return 0;
  if (check_view("sigmoid_attention", kv, heads, qk_dim, v_dim)) return 1;
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "sigmoid_attention: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  IB_CHECK_ARG(n_slices >= 1 && slice_keys >= 1 && n_slices <= 65535 && (n_slices == 1 || part), "sigmoid_attention: bad slicing %d x %d", n_slices, slice_keys);
  IB_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "sigmoid_attention: the distance bias needs both of its numbers a head");
  const long long items = (long long)T * heads;
  const dim3 grid((unsigned)((items + kWarps - 1) / kWarps), (unsigned)n_slices);
  if (act_dtype == IB_F32)
    ib::launch(sigmoid_attention_kernel<float, float>, grid, kWarps * 32, 0, stream, (const float*)q, *kv, positions, seg_of_token, scale, r1, r2, pb, (float*)out, part, T,
               heads, qk_dim, v_dim, n_slices, slice_keys, status);
  else
    ib::launch(sigmoid_attention_kernel<__nv_bfloat16, __nv_bfloat16>, grid, kWarps * 32, 0, stream, (const __nv_bfloat16*)q, *kv, positions, seg_of_token, scale, r1, r2,
               pb, (__nv_bfloat16*)out, part, T, heads, qk_dim, v_dim, n_slices, slice_keys, status);
  IB_CHECK_LAUNCH("sigmoid_attention");
  if (n_slices > 1) return ib_sigmoid_combine(part, out, act_dtype, T * heads, v_dim, n_slices, nullptr, heads, slice_keys, stream);
  return 0;
}

// 1 when the tensor-core kernel takes these sizes: bfloat16, head sizes that are multiples of 16, at most 16 query heads a kv head (a power of two or any
// divisor of 16 fills the 16 rows without a remainder; other group sizes leave rows empty).
extern "C" int ib_sigmoid_attention_mma_supports(int heads, int kv_heads, int qk_dim, int v_dim) {
  if (kv_heads <= 0 || heads % kv_heads) return 0;
  const int group = heads / kv_heads;
  return group <= 16 && qk_dim % 16 == 0 && v_dim % 16 == 0 && qk_dim <= kMaxHeadDim && v_dim <= kMaxHeadDim && sigmoid_mma_smem(qk_dim, v_dim, 16) <= 200 * 1024;
}

// How many query rows a CTA of the tensor-core kernel holds when `rows_wanted` rows of a step can share key and value tiles (the group's heads
// times the consecutive tokens of a prompt portion): 16, 32 or 64. Values above 128 columns keep 32 rows (the output's registers); two CTAs an SM
// are kept where half the rows make room for them.
extern "C" int ib_sigmoid_attention_mma_rows(int qk_dim, int v_dim, int rows_wanted) {
  int mt = v_dim > 128 ? 2 : 4;
  while (mt > 1 && (16 * (mt / 2) >= rows_wanted || sigmoid_mma_smem(qk_dim, v_dim, 16 * mt) > 200 * 1024)) mt /= 2;
  return 16 * mt;
}

extern "C" int ib_sigmoid_attention_mma(const void* q, const IbKvView* kv, const int* positions, const int* seg_of_token, const int* units, int n_units, int rows, float scale,
                                        const float* r1, const float* r2, const float* pb, void* out, float* part, int T, int heads, int qk_dim, int v_dim, int n_slices,
                                        int slice_keys, unsigned* status, cudaStream_t stream) {
  // units: null (a CTA per token and kv head) or (first token, tokens) runs of consecutive tokens of one request, at most rows / group tokens each.
  // rows: query rows a CTA holds (16, 32 or 64; see ib_sigmoid_attention_mma_rows).
  if (T == 0 || n_units == 0) return 0;
  if (check_view("sigmoid_attention_mma", kv, heads, qk_dim, v_dim)) return 1;
  IB_CHECK_ARG(kv->dtype == IB_BF16 && ib_sigmoid_attention_mma_supports(heads, kv->kv_heads, qk_dim, v_dim),
               "sigmoid_attention_mma: bfloat16 with head sizes that are multiples of 16 and at most 16 heads a kv head, got %d/%d heads of %d and %d", heads, kv->kv_heads,
               qk_dim, v_dim);
  IB_CHECK_ARG(n_slices >= 1 && slice_keys >= 1 && (n_slices == 1 || (slice_keys % kKeys == 0 && part)), "sigmoid_attention_mma: bad slicing %d x %d", n_slices, slice_keys);
  IB_CHECK_ARG(n_units <= 65535 && n_slices <= 65535, "sigmoid_attention_mma: %d units or %d slices exceed the grid limit", n_units, n_slices);
  IB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)kv->base % 16 == 0) && (kv->page_stride % 8 == 0) && (kv->v_offset % 8 == 0) && (kv->head_dim % 8 == 0),
               "sigmoid_attention_mma: pointers and rows must be 16-byte aligned");
  IB_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "sigmoid_attention_mma: the distance bias needs both of its numbers a head");
  IB_CHECK_ARG((rows == 16 || rows == 32 || rows == 64) && !(rows == 64 && v_dim > 128), "sigmoid_attention_mma: %d query rows a CTA (16, 32, or 64 up to values of 128)", rows);
  const size_t smem = sigmoid_mma_smem(qk_dim, v_dim, rows);
  IB_CHECK_ARG(smem <= 220 * 1024, "sigmoid_attention_mma: %d rows need %zu bytes of shared memory", rows, smem);
  const dim3 grid((unsigned)kv->kv_heads, (unsigned)n_units, (unsigned)n_slices);
  auto go = [&](auto kernel) {
    if (smem > 40 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kMmaWarps * 32, smem, stream, (const __nv_bfloat16*)q, *kv, positions, seg_of_token, (const int2*)units, scale, r1, r2, pb,
               (__nv_bfloat16*)out, part, heads, qk_dim, v_dim, n_slices, slice_keys, status);
  };
  if (units && rows == 64 && qk_dim <= 128 && v_dim <= 128) {   // a step with prompt portions: sixteen rows a warp
    const size_t sm = sigmoid_mma_smem(qk_dim, v_dim, 0);   // key and value tiles alone
    auto run = [&](auto kernel) {
      if (sm > 40 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      ib::launch(kernel, dim3((unsigned)kv->kv_heads, (unsigned)n_units, (unsigned)n_slices), kMmaWarps * 32, sm, stream, (const __nv_bfloat16*)q, *kv, positions,
                 seg_of_token, (const int2*)units, scale, r1, r2, pb, (__nv_bfloat16*)out, part, heads, qk_dim, v_dim, n_slices, slice_keys, status);
    };
    if (qk_dim <= 64 && v_dim <= 64) run(sigmoid_prefill_mma_kernel<4, 4>);
    else if (qk_dim <= 64) run(sigmoid_prefill_mma_kernel<4, 8>);
    else if (v_dim <= 64) run(sigmoid_prefill_mma_kernel<8, 4>);
    else run(sigmoid_prefill_mma_kernel<8, 8>);
    IB_CHECK_LAUNCH("sigmoid_prefill_mma");
    if (n_slices > 1) return ib_sigmoid_combine(part, out, IB_BF16, T * heads, v_dim, n_slices, positions, heads, slice_keys, stream);
    return 0;
  }
  const int nv = (v_dim / 16 + kMmaWarps - 1) / kMmaWarps, mtiles = rows / 16;
  auto pick = [&](auto nvc) {
    constexpr int NV = decltype(nvc)::value;
    if (mtiles == 1) go(sigmoid_attention_mma_kernel<NV, 1>);
    else if (mtiles == 2) go(sigmoid_attention_mma_kernel<NV, 2>);
    else if constexpr (NV <= 2) go(sigmoid_attention_mma_kernel<NV, 4>);
  };
  if (nv <= 1) pick(std::integral_constant<int, 1>());
  else if (nv <= 2) pick(std::integral_constant<int, 2>());
  else pick(std::integral_constant<int, 4>());
  IB_CHECK_LAUNCH("sigmoid_attention_mma");
  if (n_slices > 1) return ib_sigmoid_combine(part, out, IB_BF16, T * heads, v_dim, n_slices, nullptr, heads, slice_keys, stream);
  return 0;
}
