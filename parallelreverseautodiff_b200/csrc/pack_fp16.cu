// Packing kernels of the FP16-piece operand form (pack_fp16.cuh) and the C ABI around packed operands.
//
// One kernel produces either orientation, or both in a single pass over the source, and the source may
// be an activation evaluated on the fly (forward value, or upstream gradient times derivative): the
// operand of the next product is written where the values are born instead of being stored as FP32,
// read back, searched for its maxima and converted.  All of it is HBM-bound streaming.
//
// A CTA (256 threads = 8 warps) owns a tile of TR rows x TC columns.
//   Pass 1, one tile row per warp and trip: 128-bit loads, the activation, the optional FP32 copy; the
//   row block's maximum is a warp reduction, so the by-rows pieces of that row block are written at
//   once from registers; the values also go to a shared-memory stash (float4 stores) and every thread
//   keeps the running maximum of its columns.
//   Pass 2 (only for the by-columns form): column maxima are combined in shared memory, then each lane
//   takes one column and 32 consecutive k of it from the stash (consecutive lanes read consecutive
//   words: no bank conflicts) and writes one whole 128-byte line of pieces.
// TR is the by-columns block length, TC the by-rows block length.
#include <atomic>

#include "act_math.cuh"
#include "pack_fp16.cuh"

namespace prad {

namespace pk {

__device__ __forceinline__ float pow2f(int e) { return __int_as_float((e + 127) << 23); }

// power-of-two shift that brings a block whose largest |x| has bit pattern `absbits` into [2^14, 2^15)
__device__ __forceinline__ int shift_of(uint32_t absbits) {
  const int e = (int)((absbits >> 23) & 0xffu);
  if (e == 0 || e == 255) return 0;              // all zero / denormal, or Inf / NaN present: unscaled
  const int s = 14 - (e - 127);
  return s > PACK_SHIFT_MAX ? PACK_SHIFT_MAX : (s < PACK_SHIFT_MIN ? PACK_SHIFT_MIN : s);
}
__device__ __forceinline__ void pieces(float xs, __half& p0, __half& p1) {
  p0 = __float2half_rn(xs);
  p1 = __float2half_rn(xs - __half2float(p0));   // the difference is exact in FP32
}
__device__ __forceinline__ uint32_t absbits(float x) { return __float_as_uint(fabsf(x)); }

// the four values at (r, c .. c+3) of the source, zero outside the matrix; writes the FP32 copy
__device__ __forceinline__ void fetch4(const PackSource& s, bool vec, int64_t r, int c, int R, int C, float (&v)[4]) {
  v[0] = v[1] = v[2] = v[3] = 0.f;
  if (r >= R || c >= C) return;
  const int64_t off = r * s.ld + c;
  float a[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f}, tg[4] = {0.f, 0.f, 0.f, 0.f};
  const bool full = vec && c + 4 <= C;
  if (full) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(s.x + off));
    a[0] = t.x; a[1] = t.y; a[2] = t.z; a[3] = t.w;
    if (s.kind >= 2) {
      const float4 u = __ldcs(reinterpret_cast<const float4*>(s.dy + off));
      d[0] = u.x; d[1] = u.y; d[2] = u.z; d[3] = u.w;
    }
    if (s.kind == 3) {
      const float4 u = __ldcs(reinterpret_cast<const float4*>(s.target + off));
      tg[0] = u.x; tg[1] = u.y; tg[2] = u.z; tg[3] = u.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (c + q < C) {
        a[q] = s.x[off + q];
        if (s.kind >= 2) d[q] = s.dy[off + q];
        if (s.kind == 3) tg[q] = s.target[off + q];
      }
  }
  if (s.kind == 3) {     // MeanSquaredErrorLossOperation.Backward: scale * (output - target)
#pragma unroll
    for (int q = 0; q < 4; ++q) d[q] = mul_rn(s.loss_scale, sub_rn(d[q], tg[q]));
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (c + q >= C) continue;
    if (s.kind == 0) v[q] = a[q];
    else if (s.kind == 1) v[q] = act_value<float>((prad_act)s.act, a[q], s.act_alpha);
    else v[q] = mul_rn(d[q], act_derivative<float>((prad_act)s.act, a[q], s.act_alpha));
  }
  if (s.out) {
    if (full) __stcs(reinterpret_cast<float4*>(s.out + off), make_float4(v[0], v[1], v[2], v[3]));
    else {
#pragma unroll
      for (int q = 0; q < 4; ++q) if (c + q < C) s.out[off + q] = v[q];
    }
  }
}

// ---------------------------------------------------------------- fast path: interior 128 x 128 tiles
// The same two passes for tiles that lie completely inside the matrix, with 16-byte aligned operands and
// 128-long blocks: no bounds tests, the operation fixed at compile time, conversions two values at a
// time (cvt.rn.f16x2.f32).  OP: 0 plain; 1 / 2 / 3 forward GELU / LeakyReLU / any activation;
// 4 / 5 / 6 backward likewise; 7 / 8 mean-squared-error gradient times the GELU / any derivative;
// 9 / 10 / 11 are 1 / 4 / 7 (the GELU cases) in short arithmetic, chosen when no FP32 copy is written.
//
// Short arithmetic: the copy-less result exists only as pieces of 22 significant bits, so the GELU terms
// are contracted into fused multiply-adds and tanh is 1 - 2 / (1 + 2^(2 log2(e) u)) with the hardware's
// exp2 and reciprocal approximations (absolute error about 3e-7, of the order of the pieces' own
// rounding).  With an FP32 copy the arithmetic is the stand-alone activation kernels', operation by
// operation, so that the copy is bit-identical to theirs.
__device__ __forceinline__ void pieces2(float x0, float x1, __half2& p0, __half2& p1) {
  p0 = __floats2half2_rn(x0, x1);
  const float2 b = __half22float2(p0);
  p1 = __floats2half2_rn(x0 - b.x, x1 - b.y);      // the differences are exact in FP32
}
__device__ __forceinline__ float tanh_short(float u) {
  float t, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(u * 2.885390081777927f));    // e^(2u); inf / 0 at the ends
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t + 1.0f));
  return fmaf(-2.0f, r, 1.0f);
}
__device__ __forceinline__ float gelu_inner_short(float x, float x2) {
  return x * fmaf(x2, 0.7978845f * 0.044715f, 0.7978845f);
}
__device__ __forceinline__ float gelu_value_short(float x) {
  const float b = tanh_short(gelu_inner_short(x, x * x));
  return x * fmaf(0.5f, b, 0.5f);
}
__device__ __forceinline__ float gelu_derivative_short(float x) {
  const float x2 = x * x;
  const float b = tanh_short(gelu_inner_short(x, x2));
  const float omb2 = fmaf(-b, b, 1.0f);
  const float d = fmaf(x2, 0.7978845f * (0.044715f * 3.0f), 0.7978845f);
  return fmaf(0.5f * x, fmaf(omb2 * omb2, d, b), fmaf(0.5f, b, 0.5f));
}
template <int OP>
__device__ __forceinline__ float apply_op(const PackSource& s, float a, float d, float tg) {
  if (OP == 0) return a;
  if (OP == 1) return gelu_value<float>(a);
  if (OP == 2) return a > 0.f ? a : mul_rn(s.act_alpha, a);
  if (OP == 3) return act_value<float>((prad_act)s.act, a, s.act_alpha);
  if (OP == 9) return gelu_value_short(a);
  if (OP == 7 || OP == 8 || OP == 11) d = mul_rn(s.loss_scale, sub_rn(d, tg));
  if (OP == 4 || OP == 7) return mul_rn(d, gelu_derivative<float>(a));
  if (OP == 10 || OP == 11) return d * gelu_derivative_short(a);
  if (OP == 5) return mul_rn(d, a > 0.f ? 1.f : s.act_alpha);
  return mul_rn(d, act_derivative<float>((prad_act)s.act, a, s.act_alpha));
}

// Stash: the tile's values as floats, [128 k][128 columns] without padding; the float4 of columns 4q..4q+3
// of tile row k sits in slot q ^ ((k >> 2) & 7) of its row.  Pass 1 stores whole float4 (any permutation of
// slots is conflict-free); in pass 2 a lane reads four consecutive k of one column and the eight lanes that
// share a column quad read eight different slot positions: 32 different banks.
//
// EDGE: the one column tile that the matrix fills only in part (C is a multiple of four, so whole float4 lie inside or
// outside): columns from C on read as zeros, pieces are written up to the padded k of the by-rows form and for the
// existing operand rows of the by-columns form only.
template <int OP, bool ROWS, bool COLS, int NT, bool EDGE>
__global__ void __launch_bounds__(NT, NT == 512 ? 2 : (OP == 0 ? 5 : 3))
pack_fast_kernel(PackSource src, PackedForm fr, PackedForm fc, int tile_c0, int C) {
  constexpr int T = 128, U = 2, NW = NT / 32, NB = T / NW / U;      // NW warps, each takes every NW-th tile row
  constexpr bool HAS_DY = OP >= 4 && OP != 9, HAS_TG = OP == 7 || OP == 8 || OP == 11;
  extern __shared__ float stash[];       // [T][T] when COLS
  __shared__ unsigned colmax[T];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = (int64_t)blockIdx.y * T;
  const int ctile = tile_c0 + blockIdx.x;
  const int c0 = ctile * T, c = c0 + lane * 4;
  const bool inside = !EDGE || c < C;                  // this lane's four columns exist
  if (COLS && threadIdx.x < T) colmax[threadIdx.x] = 0;
  uint32_t cm[4] = {0, 0, 0, 0};
  // pass 1: the loads of the next two tile rows are in flight while the current two are converted
  float4 a[2][U], d[2][U], tg[2][U];
  auto load = [&](int buf, int b) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t off = (r0 + warp + NW * (b * U + u)) * src.ld + c;
      if (EDGE && !inside) {
        a[buf][u] = d[buf][u] = tg[buf][u] = make_float4(0.f, 0.f, 0.f, 0.f);
        continue;
      }
      a[buf][u] = __ldcs(reinterpret_cast<const float4*>(src.x + off));
      if (HAS_DY) d[buf][u] = __ldcs(reinterpret_cast<const float4*>(src.dy + off));
      if (HAS_TG) tg[buf][u] = __ldcs(reinterpret_cast<const float4*>(src.target + off));
    }
  };
  load(0, 0);
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    const int cur = b & 1;
    if (b + 1 < NB) load(cur ^ 1, b + 1);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tr = warp + NW * (b * U + u);
      const int64_t r = r0 + tr;
      float v[4];
      v[0] = apply_op<OP>(src, a[cur][u].x, HAS_DY ? d[cur][u].x : 0.f, HAS_TG ? tg[cur][u].x : 0.f);
      v[1] = apply_op<OP>(src, a[cur][u].y, HAS_DY ? d[cur][u].y : 0.f, HAS_TG ? tg[cur][u].y : 0.f);
      v[2] = apply_op<OP>(src, a[cur][u].z, HAS_DY ? d[cur][u].z : 0.f, HAS_TG ? tg[cur][u].z : 0.f);
      v[3] = apply_op<OP>(src, a[cur][u].w, HAS_DY ? d[cur][u].w : 0.f, HAS_TG ? tg[cur][u].w : 0.f);
      if (EDGE && !inside) v[0] = v[1] = v[2] = v[3] = 0.f;      // an activation of zero need not be zero
      if (OP >= 1 && OP <= 8 && src.out && inside)
        __stcs(reinterpret_cast<float4*>(src.out + r * src.ld + c), make_float4(v[0], v[1], v[2], v[3]));
      uint32_t m = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t bits = absbits(v[q]);
        m = max(m, bits);
        if (COLS) cm[q] = max(cm[q], bits);
      }
      if (COLS)
        *reinterpret_cast<float4*>(&stash[tr * T + ((lane ^ ((tr >> 2) & 7)) << 2)]) = make_float4(v[0], v[1], v[2], v[3]);
      if (ROWS) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        const int sh = shift_of(m);
        const float scale = pow2f(sh);
        if (lane == 0) fr.blk[(int64_t)ctile * fr.rows_ld + r] = pow2f(-sh);
        __half2 p0[2], p1[2];
        pieces2(v[0] * scale, v[1] * scale, p0[0], p1[0]);
        pieces2(v[2] * scale, v[3] * scale, p0[1], p1[1]);
        __half* dst = fr.h + r * fr.pitch + (int64_t)(c >> 5) * 64 + (c & 31);
        if (!EDGE || c < fr.kp) {                          // the row is padded with zeros up to kp and ends there
          *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(p0);
          *reinterpret_cast<uint2*>(dst + 32) = *reinterpret_cast<const uint2*>(p1);
        }
      }
    }
  }
  if (!COLS) return;
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 4; ++q)
    if (cm[q] != 0) atomicMax(&colmax[lane * 4 + q], cm[q]);
  __syncthreads();
  // pass 2: a warp owns 32 / NW quads of columns; per quad and 32-k group, lane (cc, g) converts k 4g..4g+3 of
  // column cc of the quad, and the eight lanes of a column write 64 contiguous bytes of h0 and 64 of h1:
  // whole sectors, four lines per store instruction.
  const int cc = lane & 3, g = lane >> 2;
#pragma unroll 1
  for (int quad = warp * (32 / NW); quad < (warp + 1) * (32 / NW); ++quad) {
    const int tc = quad * 4 + cc;                    // column inside the tile
    if (EDGE && c0 + quad * 4 >= C) break;           // no operand rows from here on (whole quads: C is a multiple of 4)
    const int sh = shift_of(colmax[tc]);
    const float scale = pow2f(sh);
    if (g == 0) fc.blk[(int64_t)blockIdx.y * fc.rows_ld + c0 + tc] = pow2f(-sh);
    const float* sp = stash + (4 * g) * T + (((quad ^ g) << 2) | cc);      // (k >> 2) & 7 == g for k = 32 kg + 4g + i
    __half* dst = fc.h + (int64_t)(c0 + tc) * fc.pitch + (r0 >> 5) * 64 + 4 * g;
#pragma unroll
    for (int kg = 0; kg < 4; ++kg) {
      __half2 p0[2], p1[2];
      pieces2(sp[(kg * 32) * T] * scale, sp[(kg * 32 + 1) * T] * scale, p0[0], p1[0]);
      pieces2(sp[(kg * 32 + 2) * T] * scale, sp[(kg * 32 + 3) * T] * scale, p0[1], p1[1]);
      *reinterpret_cast<uint2*>(dst + kg * 64) = *reinterpret_cast<const uint2*>(p0);
      *reinterpret_cast<uint2*>(dst + kg * 64 + 32) = *reinterpret_cast<const uint2*>(p1);
    }
  }
}

template <int OP, bool ROWS, bool COLS>
static prad_status launch_fast(prad_ctx* ctx, const PackSource& src, int tiles_r, int tiles_c, const PackedForm& fr,
                               const PackedForm& fc, int C, bool edge) {
  // with a stash (64 KB per tile) two CTAs of 16 warps hide the loads better than three of 8
  constexpr int NT = COLS ? 512 : 256;
  const int smem = COLS ? 128 * 128 * (int)sizeof(float) : 0;
  if (COLS) {
    static std::atomic<uint64_t> done{0};
    const uint64_t bit = 1ull << (ctx->device & 63);
    if (!(done.load(std::memory_order_acquire) & bit)) {
      cudaError_t e = cudaFuncSetAttribute(pack_fast_kernel<OP, ROWS, COLS, NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(pack_fast_kernel<OP, ROWS, COLS, NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("operand packing: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        return PRAD_ERR_CUDA;
      }
      done.fetch_or(bit, std::memory_order_release);
    }
  }
  if (tiles_c > 0) {
    pack_fast_kernel<OP, ROWS, COLS, NT, false><<<dim3((unsigned)tiles_c, (unsigned)tiles_r), NT, smem, ctx->stream>>>(src, fr, fc, 0, C);
    PRAD_LAUNCHED(ctx);
  }
  if (edge) {
    pack_fast_kernel<OP, ROWS, COLS, NT, true><<<dim3(1u, (unsigned)tiles_r), NT, smem, ctx->stream>>>(src, fr, fc, tiles_c, C);
    PRAD_LAUNCHED(ctx);
  }
  return PRAD_OK;
}
template <int OP>
static prad_status launch_fast_forms(prad_ctx* ctx, const PackSource& src, int tiles_r, int tiles_c, const PackedForm& fr,
                                     const PackedForm& fc, int C, bool edge) {
  if (fr.h && fc.h) return launch_fast<OP, true, true>(ctx, src, tiles_r, tiles_c, fr, fc, C, edge);
  if (fr.h) return launch_fast<OP, true, false>(ctx, src, tiles_r, tiles_c, fr, fc, C, edge);
  return launch_fast<OP, false, true>(ctx, src, tiles_r, tiles_c, fr, fc, C, edge);
}
// which compile-time operation serves this source
static int fast_op_of(const PackSource& s) {
  if (s.kind == 0) return 0;
  const bool gelu = s.act == PRAD_ACT_GELU, leaky = s.act == PRAD_ACT_LEAKY_RELU;
  if (gelu && !s.out) return s.kind == 1 ? 9 : (s.kind == 2 ? 10 : 11);
  if (s.kind == 1) return gelu ? 1 : (leaky ? 2 : 3);
  if (s.kind == 2) return gelu ? 4 : (leaky ? 5 : 6);
  return gelu ? 7 : 8;
}

template <int TR, int TC>
__global__ void __launch_bounds__(256)
pack_tile_kernel(PackSource src, bool vec, int R, int C, PackedForm fr, PackedForm fc, int fast_tiles_r, int fast_tiles_c) {
  // tiles inside the first fast_tiles_r x fast_tiles_c are written by pack_fast_kernel
  if ((int)blockIdx.y < fast_tiles_r && (int)blockIdx.x < fast_tiles_c) return;
  constexpr int W = TC / 128;            // float4 per lane and tile row
  constexpr int STRIDE = TC + 4;         // stash pitch in floats (16-byte multiple; see pass 2)
  constexpr int U = 4;                   // tile rows a warp loads before it starts converting
  extern __shared__ float stash[];       // [TR][STRIDE], only with a by-columns form
  __shared__ unsigned colmax[TC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = blockIdx.y * TR, c0 = blockIdx.x * TC;
  const bool want_rows = fr.h != nullptr, want_cols = fc.h != nullptr;
  for (int i = threadIdx.x; i < TC; i += 256) colmax[i] = 0;

  uint32_t cm[W][4];
#pragma unroll
  for (int w = 0; w < W; ++w)
#pragma unroll
    for (int q = 0; q < 4; ++q) cm[w][q] = 0;

  // ---------------------------------------------------------------- pass 1
  for (int it0 = 0; it0 < TR / 8; it0 += U) {
    float v[U][W][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = (int64_t)r0 + warp + 8 * (it0 + u);
#pragma unroll
      for (int w = 0; w < W; ++w) fetch4(src, vec, r, c0 + lane * 4 + 128 * w, R, C, v[u][w]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tr = warp + 8 * (it0 + u);
      const int64_t r = (int64_t)r0 + tr;
      uint32_t m = 0;
#pragma unroll
      for (int w = 0; w < W; ++w)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t b = absbits(v[u][w][q]);
          m = max(m, b);
          cm[w][q] = max(cm[w][q], b);
        }
      if (want_cols) {
#pragma unroll
        for (int w = 0; w < W; ++w)
          *reinterpret_cast<float4*>(&stash[tr * STRIDE + lane * 4 + 128 * w]) =
              make_float4(v[u][w][0], v[u][w][1], v[u][w][2], v[u][w][3]);
      }
      if (want_rows && r < R) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        const int sh = shift_of(m);
        const float scale = pow2f(sh);
        if (lane == 0) fr.blk[(int64_t)(c0 / TC) * fr.rows_ld + r] = pow2f(-sh);
        __half* drow = fr.h + r * fr.pitch;
#pragma unroll
        for (int w = 0; w < W; ++w) {
          const int c = c0 + lane * 4 + 128 * w;
          if (c >= fr.kp) continue;                  // beyond the padded row (kp is a multiple of 32 >= C)
          __align__(8) __half p0[4];
          __align__(8) __half p1[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) pieces(v[u][w][q] * scale, p0[q], p1[q]);
          __half* d = drow + (int64_t)(c >> 5) * 64 + (c & 31);
          *reinterpret_cast<uint2*>(d) = *reinterpret_cast<uint2*>(p0);
          *reinterpret_cast<uint2*>(d + 32) = *reinterpret_cast<uint2*>(p1);
        }
      }
    }
  }
  if (!want_cols) return;

  // ---------------------------------------------------------------- pass 2
  __syncthreads();     // colmax cleared by everybody's first statement, stash complete
#pragma unroll
  for (int w = 0; w < W; ++w)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (cm[w][q] != 0) atomicMax(&colmax[lane * 4 + 128 * w + q], cm[w][q]);
  __syncthreads();
  constexpr int CG = TC / 32, KG = TR / 32;
  for (int item = warp; item < CG * KG; item += 8) {
    const int cg = item % CG, kg = item / CG;
    const int col = c0 + cg * 32 + lane;             // operand row of the by-columns form
    const int64_t kbase = (int64_t)r0 + kg * 32;     // first k of this 32-group
    if (col >= C || kbase >= fc.kp) continue;
    const int sh = shift_of(colmax[cg * 32 + lane]);
    const float scale = pow2f(sh);
    if (kg == 0) fc.blk[(int64_t)(r0 / TR) * fc.rows_ld + col] = pow2f(-sh);
    __align__(16) __half p0[32];
    __align__(16) __half p1[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) pieces(stash[(kg * 32 + j) * STRIDE + cg * 32 + lane] * scale, p0[j], p1[j]);
    __half* d = fc.h + (int64_t)col * fc.pitch + (kbase >> 5) * 64;     // one 128-byte line: h0 | h1
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      reinterpret_cast<uint4*>(d)[j] = reinterpret_cast<const uint4*>(p0)[j];
      reinterpret_cast<uint4*>(d + 32)[j] = reinterpret_cast<const uint4*>(p1)[j];
    }
  }
}

template <int TR, int TC>
static prad_status launch_pack(prad_ctx* ctx, const PackSource& src, bool vec, int R, int C, const PackedForm& fr,
                               const PackedForm& fc, int fast_tiles_r = 0, int fast_tiles_c = 0) {
  const int smem = fc.h ? TR * (TC + 4) * (int)sizeof(float) : 0;
  if (smem > 48 * 1024) {
    static std::atomic<uint64_t> done{0};
    const uint64_t bit = 1ull << (ctx->device & 63);
    if (!(done.load(std::memory_order_acquire) & bit)) {
      const cudaError_t e = cudaFuncSetAttribute(pack_tile_kernel<TR, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("operand packing: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        return PRAD_ERR_CUDA;
      }
      done.fetch_or(bit, std::memory_order_release);
    }
  }
  // the tiles cover the padded extents: rows up to the by-columns kp, columns up to the by-rows kp
  const int64_t rows_cover = fc.h ? (fc.kp > R ? fc.kp : R) : R;
  const int64_t cols_cover = fr.h ? (fr.kp > C ? fr.kp : C) : C;
  dim3 grid((unsigned)ceil_div(cols_cover, TC), (unsigned)ceil_div(rows_cover, TR));
  PRAD_REQUIRE(grid.y <= 65535, PRAD_ERR_UNSUPPORTED, "operand packing: too many row tiles (%u)", grid.y);
  if ((int)grid.y <= fast_tiles_r && (int)grid.x <= fast_tiles_c) return PRAD_OK;    // nothing left for this kernel
  pack_tile_kernel<TR, TC><<<grid, 256, smem, ctx->stream>>>(src, vec, R, C, fr, fc, fast_tiles_r, fast_tiles_c);
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

}  // namespace pk

prad_status pack_fp16(prad_ctx* ctx, const PackSource& src, int R, int C, const PackedForm* by_rows,
                      const PackedForm* by_cols) {
  if (R <= 0 || C <= 0 || (!by_rows && !by_cols)) return PRAD_OK;
  PackedForm none;
  bool vec = (src.ld % 4 == 0) && (((uintptr_t)src.x & 15) == 0) && (!src.dy || ((uintptr_t)src.dy & 15) == 0) &&
             (!src.out || ((uintptr_t)src.out & 15) == 0) && (!src.target || ((uintptr_t)src.target & 15) == 0);
  if (by_rows) {
    PRAD_REQUIRE(by_rows->rows == R && by_rows->k == C && (by_rows->chunk == 128 || by_rows->chunk == 256), PRAD_ERR_SHAPE,
                 "operand packing: the by-rows form does not fit a %d x %d matrix", R, C);
  }
  if (by_cols) {
    PRAD_REQUIRE(by_cols->rows == C && by_cols->k == R && (by_cols->chunk == 128 || by_cols->chunk == 256), PRAD_ERR_SHAPE,
                 "operand packing: the by-columns form does not fit a %d x %d matrix", R, C);
  }
  const int tc = by_rows ? by_rows->chunk : 128, tr = by_cols ? by_cols->chunk : 128;
  if (tr == 256 && tc == 256) {
    // a 256 x 256 tile does not fit in shared memory: one pass per form (the FP32 copy is written by the first)
    prad_status s = pk::launch_pack<128, 256>(ctx, src, vec, R, C, *by_rows, none);
    if (s) return s;
    PackSource again = src;
    if (src.out) { again = PackSource(); again.kind = 0; again.x = src.out; again.ld = src.ld; }
    return pk::launch_pack<256, 128>(ctx, again, vec, R, C, none, *by_cols);
  }
  const PackedForm& fr = by_rows ? *by_rows : none;
  const PackedForm& fc = by_cols ? *by_cols : none;
  if (tr == 256) return pk::launch_pack<256, 128>(ctx, src, vec, R, C, fr, fc);
  if (tc == 256) return pk::launch_pack<128, 256>(ctx, src, vec, R, C, fr, fc);
  // 128-long blocks: interior tiles through the specialised kernel, the ragged edges through the general one
  int fr_t = 0, fc_t = 0;
  if (vec && R >= 128 && (C >= 128 || C % 4 == 0)) {
    fr_t = R / 128;
    fc_t = C / 128;
    // the last, partly filled column tile takes the same kernel when whole float4 lie inside or outside the matrix
    const bool edge = C % 128 != 0 && C % 4 == 0;
    prad_status s = PRAD_OK;
    switch (pk::fast_op_of(src)) {
      case 0: s = pk::launch_fast_forms<0>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 1: s = pk::launch_fast_forms<1>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 2: s = pk::launch_fast_forms<2>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 3: s = pk::launch_fast_forms<3>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 4: s = pk::launch_fast_forms<4>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 5: s = pk::launch_fast_forms<5>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 6: s = pk::launch_fast_forms<6>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 7: s = pk::launch_fast_forms<7>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 8: s = pk::launch_fast_forms<8>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 9: s = pk::launch_fast_forms<9>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      case 10: s = pk::launch_fast_forms<10>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
      default: s = pk::launch_fast_forms<11>(ctx, src, fr_t, fc_t, fr, fc, C, edge); break;
    }
    if (s) return s;
    if (edge) ++fc_t;
  }
  return pk::launch_pack<128, 128>(ctx, src, vec, R, C, fr, fc, fr_t, fc_t);
}

}  // namespace prad

// ---------------------------------------------------------------- C ABI
struct prad_packed {
  prad_ctx* ctx = nullptr;
  int rows = 0, cols = 0;
  prad::PackedForm by_rows, by_cols;   // h == nullptr when the form was not requested
  bool filled = false;
  uint32_t magic = 0x50414b44u;        // "PAKD"
};

using namespace prad;

namespace prad {
static bool packed_ok(const prad_packed* p) { return p && p->magic == 0x50414b44u && ctx_ok(p->ctx); }
#define PRAD_CHECK_PACKED(p, who)                                                                  \
  PRAD_REQUIRE(prad::packed_ok(p), PRAD_ERR_INVALID, who ": the packed operand is null or destroyed")

static prad_status alloc_form(PackedForm& f) {
  cudaError_t e = cudaMalloc((void**)&f.h, f.h_bytes() ? f.h_bytes() : 16);
  if (e == cudaSuccess) e = cudaMalloc((void**)&f.blk, f.blk_bytes() ? f.blk_bytes() : 16);
  if (e == cudaSuccess) e = cudaMemset(f.blk, 0, f.blk_bytes());     // rows beyond the matrix keep exponent 0
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (f.h) cudaFree(f.h);
    if (f.blk) cudaFree(f.blk);
    f.h = nullptr;
    f.blk = nullptr;
    set_error("prad_packed_create: %zu bytes could not be allocated: %s", f.h_bytes() + f.blk_bytes(), cudaGetErrorString(e));
    return PRAD_ERR_OOM;
  }
  return PRAD_OK;
}
// block length of a packed object unless the caller names one: 128 (one pass writes both forms from a
// 128 x 128 tile, three CTAs per SM), or 256 when the option "tc_chunk_k" asks for at least that
static int chunk_of(prad_ctx* ctx) { return ctx->tc_chunk_k >= 256 && ctx->tc_chunk_k_set ? 256 : 128; }
}  // namespace prad

extern "C" {

prad_status prad_packed_create(prad_ctx* ctx, int rows, int cols, int forms, int block_rows_form, int block_cols_form,
                               prad_packed** out) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_packed_create");
  PRAD_REQUIRE(out && rows > 0 && cols > 0 && (forms & 3) != 0 && (forms & ~3) == 0, PRAD_ERR_INVALID,
               "prad_packed_create: bad shape, forms must be PRAD_PACK_ROWS, PRAD_PACK_COLS or both");
  auto block_ok = [](int b) { return b == 0 || b == 128 || b == 256; };
  PRAD_REQUIRE(block_ok(block_rows_form) && block_ok(block_cols_form), PRAD_ERR_INVALID,
               "prad_packed_create: a block length is 0 (automatic), 128 or 256");
  prad_packed* p = new prad_packed();
  p->ctx = ctx;
  p->rows = rows;
  p->cols = cols;
  // both forms of one operand get different block lengths when both are wanted, so that one pass can
  // write them (a 256 x 256 tile does not fit in shared memory): the contraction over the batch (by
  // columns) keeps the long blocks
  const int chunk = chunk_of(ctx);
  prad_status s = PRAD_OK;
  if (forms & PRAD_PACK_ROWS) {
    const int b = block_rows_form ? block_rows_form : chunk;
    p->by_rows = packed_form_shape(rows, cols, b);
    s = alloc_form(p->by_rows);
  }
  if (!s && (forms & PRAD_PACK_COLS)) {
    p->by_cols = packed_form_shape(cols, rows, block_cols_form ? block_cols_form : chunk);
    s = alloc_form(p->by_cols);
  }
  if (s) {
    if (p->by_rows.h) { cudaFree(p->by_rows.h); cudaFree(p->by_rows.blk); }
    delete p;
    return s;
  }
  *out = p;
  return PRAD_OK;
}

prad_status prad_packed_destroy(prad_packed* p) {
  PRAD_CHECK_PACKED(p, "prad_packed_destroy");
  cudaStreamSynchronize(p->ctx->stream);
  for (PackedForm* f : {&p->by_rows, &p->by_cols}) {
    if (f->h) cudaFree(f->h);
    if (f->blk) cudaFree(f->blk);
  }
  p->magic = 0;
  delete p;
  return PRAD_OK;
}

static prad_status pack_into(prad_packed* p, PackSource src) {
  prad_status s = pack_fp16(p->ctx, src, p->rows, p->cols, p->by_rows.h ? &p->by_rows : nullptr,
                            p->by_cols.h ? &p->by_cols : nullptr);
  if (s == PRAD_OK) p->filled = true;
  return s;
}

prad_status prad_pack(prad_packed* p, const void* x, int64_t ld) {
  PRAD_CHECK_PACKED(p, "prad_pack");
  PRAD_CHECK_CTX(p->ctx);
  PRAD_REQUIRE(x && ld >= p->cols, PRAD_ERR_INVALID, "prad_pack: null matrix or a pitch smaller than its row length");
  PackSource src;
  src.kind = 0;
  src.x = (const float*)x;
  src.ld = ld;
  return pack_into(p, src);
}

prad_status prad_act_forward_pack(prad_packed* p, prad_act act, const void* x, void* y, double act_alpha) {
  PRAD_CHECK_PACKED(p, "prad_act_forward_pack");
  PRAD_CHECK_CTX(p->ctx);
  PRAD_REQUIRE(x && act >= PRAD_ACT_NONE && act <= PRAD_ACT_AMPLIFIED_SIGMOID, PRAD_ERR_INVALID,
               "prad_act_forward_pack: null input or unknown activation");
  PackSource src;
  src.kind = act == PRAD_ACT_NONE ? 0 : 1;
  src.x = (const float*)x;
  src.out = (float*)y;
  src.ld = p->cols;
  src.act = (int)act;
  src.act_alpha = (float)act_alpha;
  if (src.kind == 0 && y && y != x) PRAD_CUDA(cudaMemcpyAsync(y, x, (size_t)p->rows * p->cols * sizeof(float), cudaMemcpyDeviceToDevice, p->ctx->stream));
  if (src.kind == 0) src.out = nullptr;
  return pack_into(p, src);
}

prad_status prad_act_backward_pack(prad_packed* p, prad_act act, const void* saved, const void* dy, void* dx,
                                   double act_alpha) {
  PRAD_CHECK_PACKED(p, "prad_act_backward_pack");
  PRAD_CHECK_CTX(p->ctx);
  PRAD_REQUIRE(dy && act >= PRAD_ACT_NONE && act <= PRAD_ACT_AMPLIFIED_SIGMOID && (saved || act == PRAD_ACT_NONE),
               PRAD_ERR_INVALID, "prad_act_backward_pack: null input or unknown activation");
  PackSource src;
  if (act == PRAD_ACT_NONE) {
    src.kind = 0;
    src.x = (const float*)dy;
    if (dx && dx != dy) PRAD_CUDA(cudaMemcpyAsync(dx, dy, (size_t)p->rows * p->cols * sizeof(float), cudaMemcpyDeviceToDevice, p->ctx->stream));
  } else {
    src.kind = 2;
    src.x = (const float*)saved;
    src.dy = (const float*)dy;
    src.out = (float*)dx;
  }
  src.ld = p->cols;
  src.act = (int)act;
  src.act_alpha = (float)act_alpha;
  return pack_into(p, src);
}

prad_status prad_mse_act_backward_pack(prad_packed* p, prad_act act, const void* saved, const void* output, const void* target,
                                       int64_t rows_total, void* dx, double act_alpha) {
  PRAD_CHECK_PACKED(p, "prad_mse_act_backward_pack");
  PRAD_CHECK_CTX(p->ctx);
  PRAD_REQUIRE(output && target && rows_total >= 1 && act >= PRAD_ACT_NONE && act <= PRAD_ACT_AMPLIFIED_SIGMOID &&
                   (saved || act == PRAD_ACT_NONE),
               PRAD_ERR_INVALID, "prad_mse_act_backward_pack: null input, bad row count or unknown activation");
  PackSource src;
  src.kind = 3;
  src.x = (const float*)(act == PRAD_ACT_NONE ? output : saved);   // any readable tensor when there is no activation
  src.dy = (const float*)output;
  src.target = (const float*)target;
  src.loss_scale = 2.0f / (float)(rows_total * p->cols);
  src.out = (float*)dx;
  src.ld = p->cols;
  src.act = (int)act;
  src.act_alpha = (float)act_alpha;
  return pack_into(p, src);
}

prad_status prad_gemm_packed(prad_ctx* ctx, const prad_packed* A, int form_a, const prad_packed* B, int form_b,
                             double alpha, double beta, void* C, int64_t ldc, const void* bias) {
  PRAD_CHECK_CTX(ctx);
  PRAD_CHECK_PACKED(A, "prad_gemm_packed");
  PRAD_CHECK_PACKED(B, "prad_gemm_packed");
  PRAD_REQUIRE(A->ctx == ctx && B->ctx == ctx, PRAD_ERR_INVALID, "prad_gemm_packed: an operand belongs to another context");
  PRAD_REQUIRE((form_a == PRAD_PACK_ROWS || form_a == PRAD_PACK_COLS) && (form_b == PRAD_PACK_ROWS || form_b == PRAD_PACK_COLS),
               PRAD_ERR_INVALID, "prad_gemm_packed: a form is PRAD_PACK_ROWS or PRAD_PACK_COLS");
  const PackedForm& a = form_a == PRAD_PACK_ROWS ? A->by_rows : A->by_cols;
  const PackedForm& b = form_b == PRAD_PACK_ROWS ? B->by_rows : B->by_cols;
  PRAD_REQUIRE(a.h && b.h, PRAD_ERR_INVALID, "prad_gemm_packed: the operand was created without the requested form");
  PRAD_REQUIRE(A->filled && B->filled, PRAD_ERR_INVALID, "prad_gemm_packed: an operand has not been packed yet");
  PRAD_REQUIRE(a.k == b.k, PRAD_ERR_SHAPE, "Input 1 columns do not match Input 2 rows");
  PRAD_REQUIRE(a.chunk == b.chunk, PRAD_ERR_SHAPE,
               "prad_gemm_packed: the operands were packed with different block lengths (%d and %d)", a.chunk, b.chunk);
  PRAD_REQUIRE(C && ldc >= b.rows, PRAD_ERR_INVALID, "prad_gemm_packed: null result or a pitch smaller than its row length");
  return gemm_fp16x3_packed(ctx, a, b, (float)alpha, (float)beta, (float*)C, ldc, (const float*)bias);
}

prad_status prad_packed_shape(const prad_packed* p, int* rows, int* cols, int* forms, int* chunk_rows_form,
                              int* chunk_cols_form) {
  PRAD_CHECK_PACKED(p, "prad_packed_shape");
  if (rows) *rows = p->rows;
  if (cols) *cols = p->cols;
  if (forms) *forms = (p->by_rows.h ? PRAD_PACK_ROWS : 0) | (p->by_cols.h ? PRAD_PACK_COLS : 0);
  if (chunk_rows_form) *chunk_rows_form = p->by_rows.chunk;
  if (chunk_cols_form) *chunk_cols_form = p->by_cols.chunk;
  return PRAD_OK;
}

}  // extern "C"
