// Packed FP16-piece form of a float matrix: what the tensor-core FP32 GEMM (gemm_tf32x3.cu, scheme
// fp16x3) consumes.  Shared between the packing kernels (pack_fp16.cu) and the GEMM.
//
// A form holds one orientation of a matrix as a K-major operand: `rows` operand rows of `k` values.
// Every run of `chunk` consecutive k of a row (a block) is multiplied by its own power of two, chosen
// so that the block's largest magnitude lands in [2^14, 2^15), and each value is then written as two
// FP16 pieces h0 = fp16(x 2^s), h1 = fp16(x 2^s - h0): 22 significant bits.  The GEMM sums a block in
// the tensor core and multiplies the block's partial sum by 2^-s_a and 2^-s_b when it adds it to the
// running FP32 sum (one multiplication and one fused multiply-add), so the scales cost next to
// nothing and no pass over the matrix is needed to find a whole-row maximum before the first element
// can be converted.
//
// Memory layout of a row: 2*kp halves (kp = k rounded up to 32), the pieces interleaved per 32-k group,
// [h0 of k 0..31 | h1 of k 0..31 | h0 of k 32..63 | ...], so that one 128-byte TMA row brings both pieces
// of a group; padding (k..kp) is zero.  Rows are `pitch` halves apart: one 128-byte line more than the
// row needs, so that a column of lines (the same k group of consecutive rows: what a tile load reads
// and what the by-columns packing writes) does not sit at a power-of-two stride in one memory channel.
// Block scales: blk[c * rows_ld + r] = 2^-s (a float) for block c of row r; rows r >= rows hold zero.
// s is limited to [-90, 126]: values up to 2^104 keep all their bits (beyond 2^106 the pieces overflow),
// blocks whose largest magnitude is below 2^-112 lose bits; 2^-s <= 2^90 keeps the product with a
// block's partial sum (at most 2^37) finite.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace prad {

constexpr int PACK_KPAD = 32;          // k granularity of the GEMM's operand tiles
constexpr int PACK_ROWS_ALIGN = 256;   // rows_ld is a multiple of the widest output tile
constexpr int PACK_SHIFT_MIN = -90;    // limits of the power-of-two shift s of a block (see above)
constexpr int PACK_SHIFT_MAX = 126;

struct PackedForm {
  __half* h = nullptr;
  float* blk = nullptr;
  int rows = 0;       // operand rows
  int64_t k = 0;      // contraction length
  int64_t kp = 0;     // k rounded up to PACK_KPAD
  int64_t pitch = 0;  // halves between consecutive rows: 2 * kp + 64
  int rows_ld = 0;    // pitch of blk
  int nchunk = 0;     // blocks per row
  int chunk = 0;      // k per block (a multiple of 32)
  size_t h_bytes() const { return (size_t)rows * pitch * sizeof(__half); }
  size_t blk_bytes() const { return (size_t)nchunk * rows_ld * sizeof(float); }
};

inline PackedForm packed_form_shape(int rows, int64_t k, int chunk) {
  PackedForm f;
  f.rows = rows;
  f.k = k;
  f.kp = ceil_div(k, PACK_KPAD) * PACK_KPAD;
  f.pitch = 2 * f.kp + 64;
  f.rows_ld = (int)(ceil_div(rows, PACK_ROWS_ALIGN) * PACK_ROWS_ALIGN);
  f.chunk = chunk;
  f.nchunk = (int)ceil_div(f.kp, chunk);
  return f;
}

// What the packing kernel reads: a plain matrix, or an activation applied on the fly.
struct PackSource {
  int kind = 0;                   // 0 plain x ; 1 y = act(x) ; 2 dx = dy * act'(saved) ; 3 like 2 with dy = scale * (dy - target)
  const float* x = nullptr;       // plain: the matrix; forward: pre-activation; backward: saved tensor
  const float* dy = nullptr;      // backward: upstream gradient (kind 3: the network output)
  const float* target = nullptr;  // kind 3: the loss target
  float loss_scale = 0.f;         // kind 3: 2 / (rows_total * cols) of the mean squared error
  float* out = nullptr;           // optional FP32 copy of the computed values (y or dx), same pitch as x
  int64_t ld = 0;                 // pitch of x, dy and out in floats
  int act = 0;
  float act_alpha = 0.f;
};

// Packs the R x C matrix described by `src` into the requested forms (either may be null):
//   by_rows: operand rows = R, k = C (the matrix as it is);  by_cols: operand rows = C, k = R (its transpose).
prad_status pack_fp16(prad_ctx* ctx, const PackSource& src, int R, int C, const PackedForm* by_rows,
                      const PackedForm* by_cols);

// C (M x N, pitch ldc) = alpha * A B^T + beta * C for two packed operands of equal k, kp and chunk
// (gemm_tf32x3.cu).
prad_status gemm_fp16x3_packed(prad_ctx* ctx, const PackedForm& a, const PackedForm& b, float alpha, float beta,
                               float* C, int64_t ldc, const float* bias);

}  // namespace prad
