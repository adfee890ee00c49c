// Matrix products on row groups, bfloat16 on the tensor cores (m16n8k16, float32 accumulators): the products that the
// single-matrix kernels cannot take because each group of rows has its own matrix.
//
//  * grouped: the regrouped rows of routed experts (csrc/moe.cu): rows offsets[e]..offsets[e+1] go through W[e]; a 64 x 64 tile
//    belongs to one expert; the rows of x may be gathered through an index. With `gated`, W[e] holds gate rows then up rows
//    and the output is silu(gate) * up (float32 arithmetic on the accumulators).
//  * heads: out[t][b] = W[b] x[t][b] for every head b, rows and heads strided (the per-head maps around latent attention).
//
// A CTA of four warps (2 x 2, 32 x 32 each) walks K in tiles of 64 values: 16-byte cp.async copies into two swizzled buffers
// (the next tile arrives while this one is multiplied), ldmatrix fragments. Each output is one accumulation over k in a fixed
// order, so a row's result does not depend on which rows share its tile. K must be a multiple of 8 and rows 16-byte aligned.
#include <type_traits>

#include "mma_tiles.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 64;

struct RowsArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  void* out;
  // grouped
  const int* src_row;
  const int* offsets;
  const int* tile_start;
  int n_groups;
  // heads
  long long x_row, x_head, o_row, o_head;
  int rows;      // heads mode: T
  int N, K;
  int grouped;
  // heads mode: float32 partial sums [gate_P][T][gate_row], offset to the first head's column, or null: head b's output of row t is multiplied
  // by the sigmoid of its column
  const float* gate;
  int gate_P, gate_row;
  long long gate_stride;
};

template <bool GATED, typename O>
__global__ void __launch_bounds__(128) gemm_rows_mma_kernel(RowsArgs p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_g, s_r0, s_r1;
  constexpr uint32_t kA = TM * 128, kB = TN * 128, kStage = kA + (GATED ? 2 : 1) * kB;
  const uint32_t s0 = mt::smem_u32(smem);
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
  int group, r0, r1;
  if (p.grouped) {
    if (tid == 0) {
      const int b = blockIdx.y, E = p.n_groups;
      int e = -1;
      if (b < p.tile_start[E]) {
        int lo = 0, hi = E;   // the last e with tile_start[e] <= b
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (p.tile_start[mid] <= b) lo = mid;
          else hi = mid;
        }
        e = lo;
      }
      s_g = e;
      if (e >= 0) {
        s_r0 = p.offsets[e] + (b - p.tile_start[e]) * TM;
        s_r1 = p.offsets[e + 1];
      }
    }
    __syncthreads();
    group = s_g;
    if (group < 0) return;
    r0 = s_r0, r1 = s_r1;
  } else {
    group = blockIdx.z;
    r0 = blockIdx.y * TM, r1 = p.rows;
  }
  const int n0 = blockIdx.x * TN, N = p.N, K = p.K;
  const __nv_bfloat16* wg = p.w + (size_t)group * (GATED ? 2 : 1) * N * K;
  // what this thread copies: chunk (tid & 7) of rows (tid >> 3) + 16 i
  const __nv_bfloat16* a_src[4];
  const __nv_bfloat16* b_src[4];
  const __nv_bfloat16* u_src[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = (tid >> 3) + 16 * i, row = r0 + r, n = n0 + r;
    a_src[i] = nullptr;
    if (row < r1) {
      if (p.grouped) a_src[i] = p.x + (size_t)(p.src_row ? p.src_row[row] : row) * K;
      else a_src[i] = p.x + (size_t)row * p.x_row + (size_t)group * p.x_head;
    }
    b_src[i] = n < N ? wg + (size_t)n * K : nullptr;
    u_src[i] = (GATED && n < N) ? wg + (size_t)(N + n) * K : nullptr;
  }
  auto issue = [&](int kt, int buf) {
    const uint32_t sa = s0 + buf * kStage, sb = sa + kA, su = sb + kB;
    const int k = kt * TK + (tid & 7) * 8;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = (tid >> 3) + 16 * i;
      const uint32_t at = mt::tile_offset<64, TM>(r, tid & 7);
      if (a_src[i] && k < K) mt::cp_async16(sa + at, a_src[i] + k);
      else mt::st_shared_zero16(sa + at);
      if (b_src[i] && k < K) mt::cp_async16(sb + at, b_src[i] + k);
      else mt::st_shared_zero16(sb + at);
      if constexpr (GATED) {
        if (u_src[i] && k < K) mt::cp_async16(su + at, u_src[i] + k);
        else mt::st_shared_zero16(su + at);
      }
    }
    mt::cp_async_commit();
  };
  float acc[2][4][4], acu[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int a = 0; a < 2; a++)
#pragma unroll
    for (int b = 0; b < 4; b++)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        acc[a][b][c] = 0.f;
        if (GATED) acu[a % (GATED ? 2 : 1)][b][c] = 0.f;
      }
  const int nk = (K + TK - 1) / TK;
  issue(0, 0);
  for (int kt = 0; kt < nk; kt++) {
    const int buf = kt & 1;
    mt::cp_async_wait<0>();
    __syncthreads();
    if (kt + 1 < nk) issue(kt + 1, buf ^ 1);
    const uint32_t sa = s0 + buf * kStage, sb = sa + kA, su = sb + kB;
#pragma unroll
    for (int kk = 0; kk < TK / 16; kk++) {
      uint32_t a[2][4];
      mt::load_a_frag<64, TM>(sa, wm * 32, kk, lane, a[0]);
      mt::load_a_frag<64, TM>(sa, wm * 32 + 16, kk, lane, a[1]);
#pragma unroll
      for (int np = 0; np < 2; np++) {
        uint32_t r[4];
        mt::load_k_frag<64, TN>(sb, wn * 32 + 16 * np, kk, lane, r);
#pragma unroll
        for (int m = 0; m < 2; m++) {
          mt::mma_16816(acc[m][2 * np], a[m], r[0], r[1]);
          mt::mma_16816(acc[m][2 * np + 1], a[m], r[2], r[3]);
        }
        if constexpr (GATED) {
          mt::load_k_frag<64, TN>(su, wn * 32 + 16 * np, kk, lane, r);
#pragma unroll
          for (int m = 0; m < 2; m++) {
            mt::mma_16816(acu[m][2 * np], a[m], r[0], r[1]);
            mt::mma_16816(acu[m][2 * np + 1], a[m], r[2], r[3]);
          }
        }
      }
    }
  }
  O* out = (O*)p.out;
#pragma unroll
  for (int m = 0; m < 2; m++)
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int row = r0 + wm * 32 + m * 16 + g + 8 * h;
      if (row >= r1) continue;
      O* dst = p.grouped ? out + (size_t)row * N : out + (size_t)row * p.o_row + (size_t)group * p.o_head;
      float f = 1.f;
      if (!p.grouped && p.gate) {
        const float* gr = p.gate + (size_t)row * p.gate_row + group;
        float z = gr[0];
        for (int q = 1; q < p.gate_P; q++) z += gr[q * p.gate_stride];
        f = 1.f / (1.f + expf(-z));
      }
#pragma unroll
      for (int nt = 0; nt < 4; nt++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int n = n0 + wn * 32 + nt * 8 + 2 * t4 + c;
          if (n >= N) continue;
          float v = acc[m][nt][2 * h + c];
          if constexpr (GATED) v = (v / (1.f + expf(-v))) * acu[m][nt][2 * h + c];
          dst[n] = ib::from_f32<O>(v * f);
        }
    }
}

int launch_rows(const RowsArgs& a, dim3 grid, int gated, int out_dtype, cudaStream_t stream, const char* name) {
  IB_CHECK_ARG(a.K % 8 == 0 && ((uintptr_t)a.x % 16 == 0) && ((uintptr_t)a.w % 16 == 0), "%s: K = %d must be a multiple of 8 and the operands 16-byte aligned", name, a.K);
  IB_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "%s: too many row tiles or groups for one launch", name);
  auto go = [&](auto kernel, size_t smem) {
    if (smem > 40 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   // (the kernel has a few static bytes too)
    ib::launch(kernel, grid, 128, smem, stream, a);
  };
  const size_t plain = 2 * (TM + TN) * 128, gate = 2 * (TM + 2 * TN) * 128;
  if (gated && out_dtype == IB_BF16) go(gemm_rows_mma_kernel<true, __nv_bfloat16>, gate);
  else if (gated && out_dtype == IB_F32) go(gemm_rows_mma_kernel<true, float>, gate);
  else if (out_dtype == IB_BF16) go(gemm_rows_mma_kernel<false, __nv_bfloat16>, plain);
  else if (out_dtype == IB_F32) go(gemm_rows_mma_kernel<false, float>, plain);
  else return ib_set_error("%s: unknown output dtype %d", name, out_dtype);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ib_set_error("%s: %s", name, cudaGetErrorString(e));
  return 0;
}

}  // namespace

extern "C" int ib_gemm_grouped_mma(const void* x, const int* src_row, const void* w, void* out, int out_dtype, const int* offsets, const int* tile_start, int R, int E,
                                   int N, int K, int gated, cudaStream_t stream) {
  if (R == 0 || N == 0) return 0;
  IB_CHECK_ARG(R > 0 && E > 0 && N > 0 && K > 0, "gemm_grouped_mma: bad sizes rows=%d experts=%d N=%d K=%d", R, E, N, K);
  RowsArgs a = {};
  a.x = (const __nv_bfloat16*)x, a.w = (const __nv_bfloat16*)w, a.out = out, a.src_row = src_row, a.offsets = offsets, a.tile_start = tile_start;
  a.n_groups = E, a.N = N, a.K = K, a.grouped = 1;
  return launch_rows(a, dim3((N + TN - 1) / TN, R / TM + E, 1), gated, out_dtype, stream, "gemm_grouped_mma");
}

extern "C" int ib_gemm_heads_mma(const void* x, long long x_row, long long x_head, const void* w, void* out, int out_dtype, long long o_row, long long o_head, int T,
                                 int heads, int N, int K, const float* gate, int gate_P, long long gate_stride, int gate_row, cudaStream_t stream) {
  if (T == 0 || N == 0 || heads == 0) return 0;
  IB_CHECK_ARG(T > 0 && N > 0 && K > 0 && heads > 0, "gemm_heads_mma: bad sizes T=%d heads=%d N=%d K=%d", T, heads, N, K);
  IB_CHECK_ARG(x_row % 8 == 0 && x_head % 8 == 0, "gemm_heads_mma: row stride %lld and head stride %lld must be multiples of 8", x_row, x_head);
  RowsArgs a = {};
  a.x = (const __nv_bfloat16*)x, a.w = (const __nv_bfloat16*)w, a.out = out, a.x_row = x_row, a.x_head = x_head, a.o_row = o_row, a.o_head = o_head;
  a.rows = T, a.N = N, a.K = K, a.grouped = 0;
  a.gate = gate, a.gate_P = gate_P, a.gate_stride = gate_stride, a.gate_row = gate_row;
  return launch_rows(a, dim3((N + TN - 1) / TN, (T + TM - 1) / TM, heads), 0, out_dtype, stream, "gemm_heads_mma");
}
