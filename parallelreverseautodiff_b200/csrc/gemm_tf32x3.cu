// FP32 GEMM on the 5th-generation tensor cores: C = alpha*op(A)*op(B) + beta*C computed from
// split operands, accumulated in FP32 in tensor memory.  Four split schemes share the code:
//   fp16x3  (MODE 3, default): blocks of 128 or 256 k of every operand row scaled by powers of two,
//           two FP16 pieces per element, a*b ~= h1*h0' + h0*h1' + h0*h0'  (persistent kernel only;
//           operands arrive packed, see pack_fp16.cuh);
//   tf32b16 (MODE 1): a_hi*b_hi in TF32 plus two BF16 correction products;
//   tf32x3  (MODE 0): a_hi*b_hi + a_lo*b_hi + a_hi*b_lo, a_hi = tf32(a), a_lo = tf32(a - a_hi);
//   bf16x3  (MODE 2): six BF16 products of three-piece operands.
// The dropped lowest-order term is ~2^-22 relative in every scheme, so the result matches an FP32
// FMA chain to well inside the 1e-5 PRADLite tolerance.
//
// Two kernels.  gemm_tf32x3_kernel: one CTA = one 128 x 256 output tile (MODES 0, 1, 2);
// gemm_persistent_kernel: one CTA per SM walking tiles (MODES 1 and 3; see its own comment).
// Both have 320 threads:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of the operand tiles of a k-block into
//              a ring of shared-memory stages;
//   warp 1     allocates tensor memory, then one lane issues tcgen05.mma (M=128, N=256),
//              releases each stage with tcgen05.commit, and signals finished accumulators;
//   warps 2-9  epilogue: after every chunk of 256 k they tcgen05.ld that chunk's 128 x 256
//              accumulator (each warp its own 32-lane TMEM sub-partition and half of the
//              columns) and add it to running sums in registers (the tensor core truncates when
//              it adds into its accumulator; see the MMA issuer); at the end they apply the
//              power-of-two scales, alpha, beta and the bias and store.  Two TMEM accumulators
//              alternate, so chunk c+1 is multiplied while chunk c is drained.  Activations
//              are not applied here: gemm_tf32x3() runs them as separate passes.
// Both operands are consumed K-major (k contiguous).  A pre-pass writes the pieces of each operand
// into scratch in that orientation (transposing when the caller's matrix has the other
// orientation), padded so every TMA coordinate is 16-byte aligned.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the waiter raises a global
// error flag (which all other waiters poll and obey), the CTA drains, frees its tensor
// memory and returns; the host then reports PRAD_ERR_TIMEOUT.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <mutex>

#include "act_math.cuh"
#include "common.cuh"
#include "pack_fp16.cuh"

namespace prad {

namespace tc {

constexpr int BM = 128, BN = 256;
constexpr int KPAD = 32;                         // operands are padded to a multiple of this in k
constexpr int UMMA_K = 8;                        // tf32: 32 bytes per k-slice
constexpr int TMEM_COLS = 512;                   // two 128 x 256 FP32 accumulators
constexpr int CHUNK_K = 256;                     // k per accumulation chunk
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;     // producer warp, MMA warp, epilogue warps

// Pipeline shape: a k-block of BK floats is one swizzle atom wide (BK*4 = 128, 64 or 32
// bytes); STAGES k-blocks of the four operand tiles (A_hi, A_lo, B_hi, B_lo) are in flight.
// MODE 0: three TF32 products per k-slice (a_hi*b_hi + a_lo*b_hi + a_hi*b_lo), all operands
//         kept as FP32 containers.
// MODE 1: one TF32 product (a_hi*b_hi) plus the two correction products in BF16
//         (bf16(a_lo)*bf16(b) + bf16(a)*bf16(b_lo), kind::f16 with K = 16): the corrections are
//         2^-11 of the result, so BF16's 8-bit significand leaves them accurate to 2^-19 of it,
//         and they cost half a TF32 product each -- two thirds of the tensor work of MODE 0
//         for the same shared-memory footprint (4 + 2 + 2 bytes per operand element).
// MODE 2: everything in BF16: x = b0 + b1 + b2 (each piece the BF16 rounding of what is left),
//         six products b0*b0' + b0*b1' + b1*b0' + b1*b1' + b0*b2' + b2*b0' (kind::f16, K = 16).
//         The dropped terms are below 2^-24 of the result.  Same tensor work as MODE 0 but only
//         6 bytes per operand element travel from L2 to shared memory instead of 8, which is
//         what bounds this kernel (operand delivery, not the tensor pipe).
template <int BK_, int STAGES_, int MODE_ = 0> struct Cfg {
  static constexpr int BK = BK_, STAGES = STAGES_, MODE = MODE_;
  static constexpr int SWIZZLE_BYTES = BK * 4;
  static constexpr int SWIZZLE_BYTES_BF16 = BK * 2;
  static constexpr int A_TILE_BYTES = BM * BK * 4;
  static constexpr int B_TILE_BYTES = BN * BK * 4;
  // bytes per operand element in a stage: 8 (FP32 hi + FP32 lo, or FP32 hi + two BF16), or 6
  // in MODE 2 (three BF16 pieces)
  static constexpr int STAGE_BYTES = MODE == 2 ? (A_TILE_BYTES + B_TILE_BYTES) * 3 / 2
                                               : 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;
  static constexpr int CHUNK_KB = CHUNK_K / BK;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(SWIZZLE_BYTES == 128 || SWIZZLE_BYTES == 64 || SWIZZLE_BYTES == 32, "BK must be 32, 16 or 8");
  static_assert(MODE == 0 || BK >= 16, "BF16 tiles need rows of at least 32 bytes");
  static_assert(SMEM_BYTES <= 227 * 1024, "stages do not fit in shared memory");
};
constexpr uint32_t SPIN_LIMIT = 1u << 22;

// ---- raw PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive without the release (CTA scope): for hand-backs that pass no memory on.  The default arrive is a
// release, which makes the warp wait for its own outstanding stores first.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false if it gave up (own limit or somebody else's error flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err_flag, int code) {
  for (uint32_t spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 0x3ff) == 0x3ff) {
      if (*((volatile int*)err_flag) != 0) return false;
      if (spins >= SPIN_LIMIT) { atomicCAS(err_flag, 0, code); return false; }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// asks L2 for a tile of the tensor without bringing it into shared memory
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// the same wait, naming the registers of the load it completes: whatever reads them is ordered after it even
// while a later load into other registers is still in flight
__device__ __forceinline__ void tmem_ld_wait8(uint32_t (&v)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])
               :: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of SW bytes (SW = 128, 64
// or 32) with the SW-byte swizzle, i.e. what TMA writes with CU_TENSOR_MAP_SWIZZLE_{SW}B:
// 8-row groups are 8*SW bytes apart (stride byte offset), the leading byte offset is unused
// for swizzled K-major layouts, descriptor version 1 (sm_100), layout type 2 / 4 / 6 for
// the 128 / 64 / 32-byte swizzle.
template <int SW>
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t smem_addr) {
  constexpr uint64_t layout = SW == 128 ? 2 : (SW == 64 ? 4 : 6);
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;                 // leading byte offset (ignored)
  d |= (uint64_t)((8 * SW) >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;                 // version
  d |= layout << 61;
  return d;
}
// Instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = 256.
__host__ __device__ constexpr uint32_t idesc_tf32() {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = 256 (kind::f16).
__host__ __device__ constexpr uint32_t idesc_bf16() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
// Instruction descriptor: D = F32, A = B = FP16, both K-major, M = 128, N = 256 (kind::f16).
__host__ __device__ constexpr uint32_t idesc_fp16() {
  return (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

struct Epi {
  const float* bias;
  float* z_out;
  int act;
  int dact;
  const float* saved;
  float act_alpha;
  float alpha, beta;
  // operands scaled by powers of two, one scale for the whole row (unused by the packed FP16 form,
  // kept for the one-tile kernel's interface): the product of row i and column j is multiplied by
  // 2^(row_exp[i] + col_exp[j]) first; null when the operands are unscaled
  const int* row_exp;
  const int* col_exp;
  // packed FP16 operands: block scales, blk_a[c * blk_lda + i] = 2^e for block c of row i of A (likewise
  // B); the partial sum of block c is multiplied by both as it is added
  const float* blk_a = nullptr;
  const float* blk_b = nullptr;
  int blk_lda = 0, blk_ldb = 0;
};

// 2^e as a float, |e| <= 126
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((e + 127) << 23); }

// One epilogue thread's share of the finished tile: 32 consecutive columns of one row (scales,
// alpha, beta, bias; activations run as separate passes, see gemm_tf32x3).
__device__ __forceinline__ void epilogue_store32(const float (&acc)[32], int row, int col0, int M, int N,
                                                 float* __restrict__ C, int64_t ldc, bool vecC, const Epi& epi) {
  if (row >= M || col0 >= N) return;
  const int64_t off = (int64_t)row * ldc + col0;
  const bool full = vecC && (col0 + 32 <= N);
  float out[32];
  if (epi.row_exp) {   // exact: two multiplications by powers of two, each half of the exponent
    const int er = epi.row_exp[row];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int e = er + (col0 + j < N ? epi.col_exp[col0 + j] : 0);
      const int h = e >> 1;
      out[j] = epi.alpha * ((acc[j] * pow2i(h)) * pow2i(e - h));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = epi.alpha * acc[j];
  }
  if (epi.beta != 0.f) {
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = *reinterpret_cast<const float4*>(C + off + j);
        out[j] = fmaf(epi.beta, o.x, out[j]); out[j + 1] = fmaf(epi.beta, o.y, out[j + 1]);
        out[j + 2] = fmaf(epi.beta, o.z, out[j + 2]); out[j + 3] = fmaf(epi.beta, o.w, out[j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (col0 + j < N) out[j] = fmaf(epi.beta, C[off + j], out[j]);
    }
  }
  if (epi.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j) if (col0 + j < N) out[j] += epi.bias[col0 + j];
  }
  if (full) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<float4*>(C + off + j) = make_float4(out[j], out[j + 1], out[j + 2], out[j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) if (col0 + j < N) C[off + j] = out[j];
  }
}

template <class CFG>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                   const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                   const __grid_constant__ CUtensorMap map_a_x, const __grid_constant__ CUtensorMap map_b_x,
                   int M, int N, int K, float* __restrict__ C, int64_t ldc, bool vecC, Epi epi,
                   int* __restrict__ err_flag, int kb_per_split, int64_t split_stride) {
  // blockIdx.z selects a slice of the k range (split-K); slice z writes its partial product
  // to C + z * split_stride and a later pass adds the slices in order.
  // MODE 0 tiles per stage: A_hi, A_lo (FP32) | B_hi, B_lo (FP32);  map_*_x unused.
  // MODE 1 tiles per stage: A_hi (FP32), A_hb, A_lb (BF16) | B_hi (FP32), B_hb, B_lb (BF16);
  //        map_*_lo address the bf16(x - hi) arrays, map_*_x the bf16(x) arrays.
  constexpr int MODE = CFG::MODE, SWB = CFG::SWIZZLE_BYTES_BF16;
  constexpr int BK = CFG::BK, STAGES = CFG::STAGES, STAGE_BYTES = CFG::STAGE_BYTES;
  constexpr int A_TILE_BYTES = CFG::A_TILE_BYTES, B_TILE_BYTES = CFG::B_TILE_BYTES;
  constexpr int CHUNK_KB = CFG::CHUNK_KB, SW = CFG::SWIZZLE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // stage buffers must sit on a 1024-byte boundary (swizzle atom = 8 rows x 128 bytes)
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  uint8_t* generic_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(generic_base + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kb0 = blockIdx.z * kb_per_split;
  const int num_kb = min((K + BK - 1) / BK - kb0, kb_per_split);
  C += (int64_t)blockIdx.z * split_stride;
  const int num_chunks = (num_kb + CHUNK_KB - 1) / CHUNK_KB;

  // an earlier CTA gave up: do not start (one read per CTA so that all threads agree)
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = *((volatile int*)err_flag);
  __syncthreads();
  if (s_abort != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t round = kb / STAGES;
        if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, err_flag, 1)) break;
        const uint32_t st = base + s * STAGE_BYTES;
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        if (MODE == 2) {   // six BF16 tiles: A b0, b1, b2 then B b0, b1, b2
          constexpr int AT = A_TILE_BYTES / 2, BT = B_TILE_BYTES / 2;
          tma_load_2d(st, &map_a_hi, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + AT, &map_a_x, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + 2 * AT, &map_a_lo, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + 3 * AT, &map_b_hi, full_bar(s), (kb0 + kb) * BK, n0);
          tma_load_2d(st + 3 * AT + BT, &map_b_x, full_bar(s), (kb0 + kb) * BK, n0);
          tma_load_2d(st + 3 * AT + 2 * BT, &map_b_lo, full_bar(s), (kb0 + kb) * BK, n0);
          continue;
        }
        tma_load_2d(st, &map_a_hi, full_bar(s), (kb0 + kb) * BK, m0);
        tma_load_2d(st + 2 * A_TILE_BYTES, &map_b_hi, full_bar(s), (kb0 + kb) * BK, n0);
        if (MODE == 0) {
          tma_load_2d(st + A_TILE_BYTES, &map_a_lo, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + 2 * A_TILE_BYTES + B_TILE_BYTES, &map_b_lo, full_bar(s), (kb0 + kb) * BK, n0);
        } else {   // two half-size BF16 tiles where MODE 0 has one FP32 tile
          tma_load_2d(st + A_TILE_BYTES, &map_a_x, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + A_TILE_BYTES + A_TILE_BYTES / 2, &map_a_lo, full_bar(s), (kb0 + kb) * BK, m0);
          tma_load_2d(st + 2 * A_TILE_BYTES + B_TILE_BYTES, &map_b_x, full_bar(s), (kb0 + kb) * BK, n0);
          tma_load_2d(st + 2 * A_TILE_BYTES + B_TILE_BYTES + B_TILE_BYTES / 2, &map_b_lo, full_bar(s), (kb0 + kb) * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The tensor core adds each product into the FP32 accumulator with truncation, so a long
    // accumulation chain drifts towards zero.  The K loop is therefore cut into chunks of
    // CHUNK_KB k-blocks; each chunk accumulates from zero into one of two TMEM buffers and
    // the epilogue warps add finished chunks in registers with round-to-nearest.
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32();
      bool ok = true;
      for (int ch = 0; ch < num_chunks && ok; ++ch) {
        const int buf = ch & 1;
        const uint32_t use = ch >> 1;   // how many times this buffer has been used before
        if (use > 0) {
          ok = mbar_wait(acc_empty(buf), (use - 1) & 1, err_flag, 4);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        const int kb_end = min(num_kb, (ch + 1) * CHUNK_KB);
        for (int kb = ch * CHUNK_KB; kb < kb_end; ++kb) {
          const int s = kb % STAGES;
          const uint32_t round = kb / STAGES;
          ok = mbar_wait(full_bar(s), round & 1, err_flag, 2);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = base + s * STAGE_BYTES;
          const bool first_kb = kb == ch * CHUNK_KB;
          if (MODE == 2) {
            constexpr uint32_t idesc_h = idesc_bf16();
            constexpr int AT = A_TILE_BYTES / 2, BT = B_TILE_BYTES / 2;
            const uint64_t a0 = kmajor_desc<SWB>(st), a1 = kmajor_desc<SWB>(st + AT), a2 = kmajor_desc<SWB>(st + 2 * AT);
            const uint64_t b0 = kmajor_desc<SWB>(st + 3 * AT), b1 = kmajor_desc<SWB>(st + 3 * AT + BT),
                           b2 = kmajor_desc<SWB>(st + 3 * AT + 2 * BT);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {      // smallest terms first
              const uint64_t adv = (uint64_t)((k * 16 * 2) >> 4);
              umma_f16(d_tmem, a2 + adv, b0 + adv, idesc_h, !(first_kb && k == 0));
              umma_f16(d_tmem, a0 + adv, b2 + adv, idesc_h, 1);
              umma_f16(d_tmem, a1 + adv, b1 + adv, idesc_h, 1);
              umma_f16(d_tmem, a1 + adv, b0 + adv, idesc_h, 1);
              umma_f16(d_tmem, a0 + adv, b1 + adv, idesc_h, 1);
              umma_f16(d_tmem, a0 + adv, b0 + adv, idesc_h, 1);
            }
            umma_commit(empty_bar(s));
            continue;
          }
          const uint64_t a_hi = kmajor_desc<SW>(st);
          const uint64_t b_hi = kmajor_desc<SW>(st + 2 * A_TILE_BYTES);
          if (MODE == 0) {
            const uint64_t a_lo = kmajor_desc<SW>(st + A_TILE_BYTES);
            const uint64_t b_lo = kmajor_desc<SW>(st + 2 * A_TILE_BYTES + B_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);   // +32 bytes per k-slice
              umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, !(first_kb && k == 0));
              umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1);
              umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
            }
          } else {
            constexpr uint32_t idesc_h = idesc_bf16();
            const uint64_t a_hb = kmajor_desc<SWB>(st + A_TILE_BYTES);
            const uint64_t a_lb = kmajor_desc<SWB>(st + A_TILE_BYTES + A_TILE_BYTES / 2);
            const uint64_t b_hb = kmajor_desc<SWB>(st + 2 * A_TILE_BYTES + B_TILE_BYTES);
            const uint64_t b_lb = kmajor_desc<SWB>(st + 2 * A_TILE_BYTES + B_TILE_BYTES + B_TILE_BYTES / 2);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {      // BF16 slices are 16 wide = 32 bytes
              const uint64_t adv = (uint64_t)((k * 16 * 2) >> 4);
              umma_f16(d_tmem, a_lb + adv, b_hb + adv, idesc_h, !(first_kb && k == 0));
              umma_f16(d_tmem, a_hb + adv, b_lb + adv, idesc_h, 1);
            }
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
              umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
            }
          }
          umma_commit(empty_bar(s));   // the stage may be refilled once these MMAs have read it
        }
        umma_commit(acc_full(buf));    // chunk complete (arrives even after a give-up)
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int sub = warp & 3;                 // TMEM sub-partition this warp may read
    const int half = (warp - 2) >> 2;         // which 128 columns of the tile
    const int row = m0 + sub * 32 + lane;
    float sum[4][32];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
      for (int j = 0; j < 32; ++j) sum[g][j] = 0.f;
    bool ok = true;
    for (int ch = 0; ch < num_chunks && ok; ++ch) {
      const int buf = ch & 1;
      ok = mbar_wait(acc_full(buf), (ch >> 1) & 1, err_flag, 3);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(buf * BN + half * 128);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t v[32];
        tmem_ld32(taddr + (uint32_t)(g * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[g][j] = __fadd_rn(sum[g][j], __uint_as_float(v[j]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
    }
    if (ok && *((volatile int*)err_flag) == 0) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        epilogue_store32(sum[g], row, n0 + half * 128 + g * 32, M, N, C, ldc, vecC, epi);
    }
  }

  // drain: nobody leaves while tensor-core work or bulk copies of this CTA may be in flight.
  // In the normal path every issued TMA load was consumed by an MMA and every MMA was
  // waited for through acc_full before the last chunk was read.
  tc_fence_before();
  __syncthreads();
  if (*((volatile int*)err_flag) != 0) {
    // give-up path: bulk copies or MMAs issued before the give-up may still be running;
    // they finish within microseconds, so a fixed, bounded pause covers them
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- quad-transposed epilogue -----------------------------------------------------------
// After the accumulator is drained a lane holds 32 consecutive columns of ONE row per group, so
// a direct 16-byte store touches 32 different rows per instruction.  Two butterfly exchanges
// inside each quad of lanes (xor 2, then xor 1; registers only, the shared-memory pipe belongs
// to the tensor core) re-deal a 32-column group so that lane i of quad q holds, for each of
// the quad's four rows s, the columns 4 (i + 4 h) .. + 3 (h = 0, 1): the four lanes of a quad
// then write 64 contiguous bytes of one row, and an instruction touches 8 rows instead of 32.
// The epilogue applies the power-of-two scales, alpha, beta and the bias; activations run as a
// separate pass (see gemm_tf32x3), which also keeps this fully unrolled code small.
__device__ __forceinline__ void quad_transpose(float (&v)[32], int lane) {
  const bool hi2 = (lane & 2) != 0, hi1 = (lane & 1) != 0;
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int k = 0; k < 4; ++k) {     // column blocks c and c + 2 against lane ^ 2
        float& lo = v[4 * (c + 4 * h) + k];
        float& hi = v[4 * (c + 2 + 4 * h) + k];
        const float recv = __shfl_xor_sync(0xffffffffu, hi2 ? lo : hi, 2);
        if (hi2) lo = recv; else hi = recv;
      }
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int k = 0; k < 4; ++k) {     // slots 2u and 2u + 1 against lane ^ 1
        float& lo = v[4 * (2 * u + 4 * h) + k];
        float& hi = v[4 * (2 * u + 1 + 4 * h) + k];
        const float recv = __shfl_xor_sync(0xffffffffu, hi1 ? lo : hi, 1);
        if (hi1) lo = recv; else hi = recv;
      }
  // now v[4 (s + 4 h) + k] = row 4 (lane / 4) + s, column 4 ((lane & 3) + 4 h) + k of the group
}

__device__ __forceinline__ void epilogue_quad(float o0, float o1, float o2, float o3, int row, int c, int er, int M,
                                              int N, float* __restrict__ C, int64_t ldc, bool vecC, const Epi& epi) {
  if (row >= M || c >= N) return;
  const int64_t off = (int64_t)row * ldc + c;
  const bool full = vecC && (c + 4 <= N);
  float o[4] = {o0, o1, o2, o3};
  if (epi.row_exp) {   // exact: two multiplications by powers of two, each half of the exponent
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = er + (c + q < N ? epi.col_exp[c + q] : 0);
      const int h = e >> 1;
      o[q] = epi.alpha * ((o[q] * pow2i(h)) * pow2i(e - h));
    }
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = epi.alpha * o[q];
  }
  if (epi.beta != 0.f) {
    if (full) {
      const float4 old = *reinterpret_cast<const float4*>(C + off);
      o[0] = fmaf(epi.beta, old.x, o[0]); o[1] = fmaf(epi.beta, old.y, o[1]);
      o[2] = fmaf(epi.beta, old.z, o[2]); o[3] = fmaf(epi.beta, old.w, o[3]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) if (c + q < N) o[q] = fmaf(epi.beta, C[off + q], o[q]);
    }
  }
  if (epi.bias) {
#pragma unroll
    for (int q = 0; q < 4; ++q) if (c + q < N) o[q] += epi.bias[c + q];
  }
  if (full) {
    __stcs(reinterpret_cast<float4*>(C + off), make_float4(o[0], o[1], o[2], o[3]));
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) if (c + q < N) C[off + q] = o[q];
  }
}

// sum[g][j] = column col0 + 32 g + j of row row0 + lane (modified in place)
__device__ __forceinline__ void epilogue_store_warp(float (&sum)[4][32], int lane, int row0, int col0, int M, int N,
                                                    float* __restrict__ C, int64_t ldc, bool vecC, const Epi& epi) {
  const int qrow = row0 + 4 * (lane >> 2), i = lane & 3;
  // A tile inside the matrix with a plain epilogue (nearly every store of a large product): no bounds tests, no
  // per-quad address arithmetic -- four row pointers and immediate offsets.  This is about instruction fetch, not about
  // executed work: the straight-line store code runs once per tile, so it is fetched anew every time, and the warps
  // waited for instructions more than for anything else while it ran (warp state statistics of a short-k product:
  // "no instruction" four cycles per issued instruction).  The general path below is three times as long.
  // (Columns: the warp's 128 or, at the right edge, a multiple of 16, so that each store instruction is all or nothing.)
  const int ncols = N - col0 < 128 ? N - col0 : 128;
  if (ncols <= 0 || row0 >= M) return;
  if (vecC && epi.beta == 0.f && !epi.bias && !epi.row_exp && row0 + 32 <= M && (ncols & 15) == 0) {
    float* rp[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) rp[s] = C + (int64_t)(qrow + s) * ldc + col0 + 4 * i;
    if (epi.alpha != 1.f) {
      const float alpha = epi.alpha;
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[g][j] = alpha * sum[g][j];
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (32 * g >= ncols) break;
      quad_transpose(sum[g], lane);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (32 * g + 16 * h >= ncols) break;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int j = 4 * (s + 4 * h);
          __stcs(reinterpret_cast<float4*>(rp[s] + 32 * g + 16 * h),
                 make_float4(sum[g][j], sum[g][j + 1], sum[g][j + 2], sum[g][j + 3]));
        }
      }
    }
    return;
  }
  int er[4] = {0, 0, 0, 0};
  if (epi.row_exp) {
#pragma unroll
    for (int s = 0; s < 4; ++s) er[s] = qrow + s < M ? epi.row_exp[qrow + s] : 0;
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    quad_transpose(sum[g], lane);
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int j = 4 * (s + 4 * h);
        epilogue_quad(sum[g][j], sum[g][j + 1], sum[g][j + 2], sum[g][j + 3], qrow + s,
                      col0 + 32 * g + 4 * (i + 4 * h), er[s], M, N, C, ldc, vecC, epi);
      }
  }
}

// ---- persistent variant of MODE 1 (TF32 product + two BF16 corrections) -----------------
// Same arithmetic and tile as gemm_tf32x3_kernel<Cfg<32,2,1>>, organised differently:
//   * one CTA per SM walks output tiles (n-tile fastest, then m-tile, then k-slice): its
//     first tile is blockIdx.x, every further one comes from a global counter
//     (gridDim.x + atomicAdd), so a CTA that starts late -- its SM was busy with a
//     collective's kernel, say -- simply takes fewer tiles.  The producer publishes each
//     tile index to the other warps through a four-entry queue in shared memory.  The
//     epilogue warps store tile i while the producer and MMA warps already work on tile
//     i+1 (the two TMEM accumulators decouple them by two 256-k chunks).  Which CTA
//     computes a tile does not change its result.  The last CTA to finish resets the
//     counters for the next launch;
//   * the operand ring holds four units of 48 KB instead of two stages of 96 KB, each with its
//     own full/empty barrier pair, so a unit is refilled as soon as the MMAs that read it retire
//     and three loads are in flight while one is multiplied.  PMODE 1: a k-block of 32 arrives
//     as unit H (the four BF16 tiles a_hb, a_lb, b_hb, b_lb) and unit F (the two FP32 tiles
//     a_hi, b_hi).  PMODE 3: a k-block of 32 is one unit of two tiles whose 128-byte rows hold
//     both FP16 pieces of a row (h0 | h1): two TMA instructions and 384 row requests per unit --
//     with four tiles of 64-byte rows the TMA unit's request rate, not its bytes, held the kernel
//     back (4 % slower; adding L2 prefetch requests on top cost another 10 %).
namespace p1 {
constexpr int BK = 32;
constexpr int UNITS = 4;
constexpr int UNIT_BYTES = 48 * 1024;
constexpr int CHUNK_KB = CHUNK_K / BK;
constexpr int SCALE_BYTES = EPI_WARPS * 128 * 4;   // PMODE 3: each epilogue warp's copy of its 128 column scales of a block
constexpr int SMEM_BYTES = UNITS * UNIT_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + SCALE_BYTES;
static_assert(SMEM_BYTES <= 227 * 1024, "unit ring does not fit in shared memory");
}  // namespace p1

struct TileSched {
  int tiles_m, tiles_n, splits;   // tile t -> (t % tiles_n, (t / tiles_n) % tiles_m, t / (tiles_n * tiles_m))
  int kb_per_split, total_kb;     // k-blocks per slice and in all
  int chunk_kb;                   // k-blocks per accumulation chunk
  int panel_n;                    // column tiles per panel of the tile walk
  int64_t split_stride;           // elements between the partial products of consecutive slices
  int prefetch_kb;                // PMODE 3: k-blocks by which an L2 prefetch of the row operand runs ahead of its load (0 = none)
};

template <int PMODE>
__global__ void __launch_bounds__(THREADS, 1)   // 10 warps, at most 3 per scheduler: 3 x 32 x 168 registers fit its 16 K file
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_xb,
                               const __grid_constant__ CUtensorMap map_a_lb, const __grid_constant__ CUtensorMap map_b_hi,
                               const __grid_constant__ CUtensorMap map_b_xb, const __grid_constant__ CUtensorMap map_b_lb,
                               int M, int N, float* __restrict__ C, int64_t ldc, bool vecC, Epi epi,
                               int* __restrict__ err_flag, TileSched ts) {
  using namespace p1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + UNITS * UNIT_BYTES;
  auto full_bar = [&](uint32_t s) { return bars + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bars + 8u * (UNITS + s); };
  auto acc_full = [&](uint32_t b) { return bars + 8u * (2 * UNITS + b); };
  auto acc_empty = [&](uint32_t b) { return bars + 8u * (2 * UNITS + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * UNITS + 4);
  constexpr int TQ = 4;                       // depth of the tile-index queue
  auto tile_full = [&](uint32_t i) { return bars + 8u * (2 * UNITS + 5 + i); };
  auto tile_empty = [&](uint32_t i) { return bars + 8u * (2 * UNITS + 5 + TQ + i); };
  uint8_t* generic_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(generic_base + UNITS * UNIT_BYTES + 8 * (2 * UNITS + 4));
  volatile int* tile_q =
      reinterpret_cast<volatile int*>(generic_base + UNITS * UNIT_BYTES + 8 * (2 * UNITS + 5 + 2 * TQ));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = ts.tiles_m * ts.tiles_n * ts.splits;
  int* const tile_counter = err_flag + 32;    // tiles handed out beyond the first gridDim.x
  int* const done_counter = err_flag + 33;    // CTAs that have finished

  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = *((volatile int*)err_flag);
  __syncthreads();
  if (s_abort != 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < UNITS; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), EPI_WARPS); }
    for (int i = 0; i < TQ; ++i) { mbar_init(tile_full(i), 1); mbar_init(tile_empty(i), 1 + EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // consumers: next tile index from the queue (-1 = no more tiles, -2 = gave up)
  // (whole_warp: called by all 32 lanes, which then agree on the outcome)
  auto next_tile = [&](uint32_t qi, int role, bool whole_warp) -> int {
    const uint32_t slot = qi % TQ;
    bool got = mbar_wait(tile_full(slot), (qi / TQ) & 1, err_flag, role);
    if (whole_warp) got = __all_sync(0xffffffffu, got);
    if (!got) return -2;
    const int t = tile_q[slot];
    if (whole_warp) __syncwarp();
    if (lane == 0) mbar_arrive(tile_empty(slot));
    return t;
  };

  // tile t of this CTA: origin of the output tile and its k range
  // Tiles are walked panel by panel: all row tiles of `panel_n` column tiles before the next panel, so
  // that the column operand of a panel stays in L2 while the row operand streams past it.
  auto tile_of = [&](int t, int& m0, int& n0, int& z, int& kb0, int& num_kb) {
    const int per_slice = ts.tiles_n * ts.tiles_m;
    z = t / per_slice;
    const int t2 = t - z * per_slice;
    const int p = t2 / (ts.tiles_m * ts.panel_n);
    const int r = t2 - p * ts.tiles_m * ts.panel_n;
    const int w = min(ts.panel_n, ts.tiles_n - p * ts.panel_n);
    m0 = (r / w) * BM;
    n0 = (p * ts.panel_n + r % w) * BN;
    kb0 = z * ts.kb_per_split;
    num_kb = min(ts.total_kb - kb0, ts.kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t g = 0;    // units issued so far, over all tiles of this CTA
      uint32_t qi = 0;   // tile indices published so far
      bool ok = true;
      int t = blockIdx.x;
      while (ok) {
        const uint32_t qslot = qi % TQ, qround = qi / TQ;
        if (qround > 0 && !mbar_wait(tile_empty(qslot), (qround - 1) & 1, err_flag, 5)) break;
        tile_q[qslot] = t < total_tiles ? t : -1;
        mbar_arrive(tile_full(qslot));        // release: the entry is visible to whoever sees the phase
        ++qi;
        if (t >= total_tiles) break;
        int m0, n0, z, kb0, num_kb;
        tile_of(t, m0, n0, z, kb0, num_kb);
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          const int x = (kb0 + kb) * BK;
#pragma unroll
          for (int half = 0; half < (PMODE == 1 ? 2 : 1); ++half, ++g) {
            const uint32_t slot = g & (UNITS - 1), round = g / UNITS;
            if (round > 0 && !mbar_wait(empty_bar(slot), (round - 1) & 1, err_flag, 1)) { ok = false; break; }
            const uint32_t st = base + slot * UNIT_BYTES;
            mbar_expect_tx(full_bar(slot), UNIT_BYTES);
            if (PMODE == 3) {  // one unit: A rows (h0 | h1) 16 KB, B rows (h0 | h1) 32 KB; x counts halves
              tma_load_2d(st, &map_a_xb, full_bar(slot), 2 * x, m0);
              tma_load_2d(st + 16 * 1024, &map_b_xb, full_bar(slot), 2 * x, n0);
              // the row operand streams from DRAM: its tile of a later k-block is requested into L2 now
              if (ts.prefetch_kb > 0 && kb + ts.prefetch_kb < num_kb) tma_prefetch_2d(&map_a_xb, 2 * (x + ts.prefetch_kb * BK), m0);
            } else if (half == 0) {   // unit H: a_hb 8 KB | a_lb 8 KB | b_hb 16 KB | b_lb 16 KB
              tma_load_2d(st, &map_a_xb, full_bar(slot), x, m0);
              tma_load_2d(st + 8 * 1024, &map_a_lb, full_bar(slot), x, m0);
              tma_load_2d(st + 16 * 1024, &map_b_xb, full_bar(slot), x, n0);
              tma_load_2d(st + 32 * 1024, &map_b_lb, full_bar(slot), x, n0);
            } else {           // unit F: a_hi 16 KB | b_hi 32 KB
              tma_load_2d(st, &map_a_hi, full_bar(slot), x, m0);
              tma_load_2d(st + 16 * 1024, &map_b_hi, full_bar(slot), x, n0);
            }
          }
        }
        t = (int)gridDim.x + atomicAdd(tile_counter, 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(), idesc_h = idesc_bf16();
      uint32_t g = 0, gc = 0, qi = 0;   // units consumed, chunks started, tiles taken
      bool ok = true;
      // -DPRAD_GEMM_STALL_PROBE: cycle counts of what this thread and one epilogue warp wait for, printed by
      // CTA 0 at the end of every launch (a diagnostic build; the numbers quoted in the design notes come from it)
#ifdef PRAD_GEMM_STALL_PROBE
      long long w_full = 0, w_acc = 0, w_tile = 0;
      const long long t_begin = clock64();
#define PROBE_WAIT(acc, expr) { const long long p0_ = clock64(); expr; acc += clock64() - p0_; }
#else
#define PROBE_WAIT(acc, expr) { expr; }
#endif
      while (ok) {
        int t;
        PROBE_WAIT(w_tile, t = next_tile(qi++, 6, false));
        if (t < 0) break;
        int m0, n0, z, kb0, num_kb;
        tile_of(t, m0, n0, z, kb0, num_kb);
        const int num_chunks = (num_kb + ts.chunk_kb - 1) / ts.chunk_kb;
        for (int ch = 0; ch < num_chunks && ok; ++ch, ++gc) {
          const uint32_t buf = gc & 1, use = gc >> 1;
          if (use > 0) {
            PROBE_WAIT(w_acc, ok = mbar_wait(acc_empty(buf), (use - 1) & 1, err_flag, 4));
            if (!ok) break;
            tc_fence_after();
          }
          const uint32_t d_tmem = tmem_base + buf * (uint32_t)BN;
          const int kb_end = min(num_kb, (ch + 1) * ts.chunk_kb);
          for (int kb = ch * ts.chunk_kb; kb < kb_end && ok; ++kb) {
            if (PMODE == 3) {   // one unit: A (h0 | h1 per row), B likewise; three FP16 products, smallest first
              constexpr uint32_t idesc_q = idesc_fp16();
              const uint32_t slot = g & (UNITS - 1);
              PROBE_WAIT(w_full, ok = mbar_wait(full_bar(slot), (g / UNITS) & 1, err_flag, 2));
              if (!ok) break;
              tc_fence_after();
              const uint32_t st = base + slot * UNIT_BYTES;
              // rows of 128 bytes (128-byte swizzle): h0 at byte 0, h1 at byte 64, 16-k slices 32 bytes apart
              const uint64_t a_0 = kmajor_desc<128>(st), a_1 = a_0 + 4;
              const uint64_t b_0 = kmajor_desc<128>(st + 16 * 1024), b_1 = b_0 + 4;
#pragma unroll
              for (int k = 0; k < BK / 16; ++k) {
                const uint64_t adv = (uint64_t)((k * 16 * 2) >> 4);
                umma_f16(d_tmem, a_1 + adv, b_0 + adv, idesc_q, !(kb == ch * ts.chunk_kb && k == 0));
                umma_f16(d_tmem, a_0 + adv, b_1 + adv, idesc_q, 1);
                umma_f16(d_tmem, a_0 + adv, b_0 + adv, idesc_q, 1);
              }
              umma_commit(empty_bar(slot));
              ++g;
              continue;
            }
            {   // unit H: the two BF16 correction products, two 16-wide k-slices
              const uint32_t slot = g & (UNITS - 1);
              ok = mbar_wait(full_bar(slot), (g / UNITS) & 1, err_flag, 2);
              if (!ok) break;
              tc_fence_after();
              const uint32_t st = base + slot * UNIT_BYTES;
              const uint64_t a_hb = kmajor_desc<64>(st), a_lb = kmajor_desc<64>(st + 8 * 1024);
              const uint64_t b_hb = kmajor_desc<64>(st + 16 * 1024), b_lb = kmajor_desc<64>(st + 32 * 1024);
#pragma unroll
              for (int k = 0; k < BK / 16; ++k) {
                const uint64_t adv = (uint64_t)((k * 16 * 2) >> 4);
                umma_f16(d_tmem, a_lb + adv, b_hb + adv, idesc_h, !(kb == ch * ts.chunk_kb && k == 0));
                umma_f16(d_tmem, a_hb + adv, b_lb + adv, idesc_h, 1);
              }
              umma_commit(empty_bar(slot));
              ++g;
            }
            {   // unit F: the TF32 product, four 8-wide k-slices
              const uint32_t slot = g & (UNITS - 1);
              ok = mbar_wait(full_bar(slot), (g / UNITS) & 1, err_flag, 2);
              if (!ok) break;
              tc_fence_after();
              const uint32_t st = base + slot * UNIT_BYTES;
              const uint64_t a_hi = kmajor_desc<128>(st), b_hi = kmajor_desc<128>(st + 16 * 1024);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
                umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1);
              }
              umma_commit(empty_bar(slot));
              ++g;
            }
          }
          umma_commit(acc_full(buf));    // chunk complete (arrives even after a give-up)
        }
      }
#ifdef PRAD_GEMM_STALL_PROBE
      if (blockIdx.x == 0)
        printf("mma issuer: total %lld cycles, waited for operands %lld, for the accumulator %lld, for tiles %lld (units %u)\n",
               clock64() - t_begin, w_full, w_acc, w_tile, g);
#endif
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int sub = warp & 3;                 // TMEM sub-partition this warp may read
    const int half = (warp - 2) >> 2;         // which 128 columns of the tile
    uint32_t gc = 0, qi = 0;
    bool ok = true;
#ifdef PRAD_GEMM_STALL_PROBE
    long long e_wait = 0, e_drain = 0, e_store = 0;
    const long long e_begin = clock64();
#endif
    while (ok) {
      const int t = next_tile(qi++, 7, true);
      if (t < 0) break;
      int m0, n0, z, kb0, num_kb;
      tile_of(t, m0, n0, z, kb0, num_kb);
      const int num_chunks = (num_kb + ts.chunk_kb - 1) / ts.chunk_kb;
      float sum[4][32];
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[g][j] = 0.f;
      // packed FP16 operands: block c of this slice is block kb0 / chunk_kb + c of the operands
      const int chunk0 = kb0 / ts.chunk_kb;
      const int row_blk = min(m0 + sub * 32 + lane, M - 1);     // rows beyond M are never stored
      // PMODE 3: the scales of the next block are fetched while the current one is summed -- this thread's row
      // scale into a register, the 128 column scales one float4 per lane; at the start of a block the lanes
      // put theirs into the warp's slot of shared memory, from where every lane reads all of them (broadcast)
      float sa_next = 0.f;
      float4 sb_next = make_float4(0.f, 0.f, 0.f, 0.f);
      float4* const sb_slot = reinterpret_cast<float4*>(generic_base + UNITS * UNIT_BYTES + 256) + (warp - 2) * 32;
      auto fetch_scales = [&](int ch) {
        sa_next = __ldg(epi.blk_a + (int64_t)(chunk0 + ch) * epi.blk_lda + row_blk);
        sb_next = __ldg(reinterpret_cast<const float4*>(epi.blk_b + (int64_t)(chunk0 + ch) * epi.blk_ldb + n0 + half * 128) + lane);
      };
      if (PMODE == 3) fetch_scales(0);
      for (int ch = 0; ch < num_chunks; ++ch, ++gc) {
        const uint32_t buf = gc & 1;
        float sa = 0.f;
        if (PMODE == 3) {
          sa = sa_next;
          sb_slot[lane] = sb_next;      // the previous block's readers passed the __syncwarp at its end
          __syncwarp();
          if (ch + 1 < num_chunks) fetch_scales(ch + 1);
        }
#ifdef PRAD_GEMM_STALL_PROBE
        const long long c1_ = clock64();
#endif
        ok = __all_sync(0xffffffffu, mbar_wait(acc_full(buf), (gc >> 1) & 1, err_flag, 3));
        if (!ok) break;
        tc_fence_after();
#ifdef PRAD_GEMM_STALL_PROBE
        const long long c2_ = clock64();
        e_wait += c2_ - c1_;
#endif
        const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + buf * (uint32_t)BN + (uint32_t)(half * 128);
        if (PMODE == 3) {
          // eight columns per load, the next load in flight while the current eight are added: the live
          // registers stay at 128 running sums + two loads
          const float2 sa2 = make_float2(sa, sa);
          uint32_t v[2][8];
          tmem_ld8(taddr, v[0]);
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            uint32_t (&cur)[8] = v[g & 1];
            tmem_ld_wait8(cur);
            if (g + 1 < 16) tmem_ld8(taddr + (uint32_t)((g + 1) * 8), v[(g + 1) & 1]);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const float4 t = sb_slot[g * 2 + q];
              float* acc = &sum[g >> 2][(g & 3) * 8 + 4 * q];
              // sum += (partial * 2^e_a) * 2^e_b: the first product is exact, the sum is rounded once;
              // two columns per instruction (packed FP32)
              const float2 p01 = __fmul2_rn(make_float2(__uint_as_float(cur[4 * q]), __uint_as_float(cur[4 * q + 1])), sa2);
              const float2 p23 = __fmul2_rn(make_float2(__uint_as_float(cur[4 * q + 2]), __uint_as_float(cur[4 * q + 3])), sa2);
              const float2 r01 = __ffma2_rn(p01, make_float2(t.x, t.y), make_float2(acc[0], acc[1]));
              const float2 r23 = __ffma2_rn(p23, make_float2(t.z, t.w), make_float2(acc[2], acc[3]));
              acc[0] = r01.x; acc[1] = r01.y; acc[2] = r23.x; acc[3] = r23.y;
            }
          }
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t v[32];
            tmem_ld32(taddr + (uint32_t)(g * 32), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[g][j] = __fadd_rn(sum[g][j], __uint_as_float(v[j]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_relaxed(acc_empty(buf));     // (the TMEM reads are ordered by the tcgen05 fence)
#ifdef PRAD_GEMM_STALL_PROBE
        e_drain += clock64() - c2_;
#endif
      }
#ifdef PRAD_GEMM_STALL_PROBE
      const long long st0_ = clock64();
#endif
      if (!ok) break;
      // has another CTA given up?  Asked before the stores and looked at after them: the answer takes a trip to L2
      const int gave_up = *((volatile int*)err_flag);
      float* Ct = C + (int64_t)z * ts.split_stride;
      epilogue_store_warp(sum, lane, m0 + sub * 32, n0 + half * 128, M, N, Ct, ldc, vecC, epi);
      if (gave_up != 0) { ok = false; break; }
#ifdef PRAD_GEMM_STALL_PROBE
      e_store += clock64() - st0_;
#endif
    }
#ifdef PRAD_GEMM_STALL_PROBE
    if (blockIdx.x == 0 && warp == 2 && lane == 0)
      printf("epilogue warp: total %lld cycles, tiles %u, blocks %u: waited for a block %lld, summed blocks %lld, stored tiles %lld\n",
             clock64() - e_begin, qi - 1, gc, e_wait, e_drain, e_store);
#endif
  }

  // drain, as in the one-tile kernel
  tc_fence_before();
  __syncthreads();
  if (*((volatile int*)err_flag) != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  // the last CTA to get here (every producer has drawn its final index by then) zeroes the
  // counters for the next launch on this stream
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1) == (int)gridDim.x - 1) {
      *((volatile int*)tile_counter) = 0;
      *((volatile int*)done_counter) = 0;
      __threadfence();
    }
  }
}

// ---- CTA-pair variant of the packed FP16 product (tcgen05 cta_group::2) --------------------
// Two CTAs on neighbouring SMs (a cluster of two) share one 256 x 256 output tile: each holds 128 rows of
// the row operand and HALF of the column operand's 256 rows in its shared memory, the tensor cores of both
// SMs read both halves, and each CTA's TMEM receives its own 128 x 256 part of the product.  Per SM and
// k-block that is 32 KB of operands instead of 48 KB: less traffic from L2 and through shared memory, and
// six units fit where four did, so five loads are in flight while one is multiplied.
//   * the even CTA of the pair (rank 0, "leader") draws the tile indices, issues every MMA and owns the
//     barriers both CTAs report to: unit filled (`full`: the leader announces the bytes of both CTAs, both
//     CTAs' TMA loads complete on it), accumulator drained (`acc_empty`: the epilogue warps of both CTAs
//     arrive), queue entry consumed (`tile_empty`).  What the leader tells the pair -- unit free again,
//     accumulator ready, next tile index -- it signals on the barrier of the same name in EACH CTA
//     (two tcgen05.commit, or a remote store + remote arrive for the queue);
//   * every CTA loads its own operand rows, drains its own TMEM rows and stores its own output rows;
//   * the pair synchronises (barrier.cluster) after the barriers are initialised and before TMEM is freed,
//     so no remote arrive meets an uninitialised barrier or a CTA that has left.
//   * the accumulator hand-back of the other CTA's epilogue warps is a RELAXED remote arrive: with a release at
//     cluster scope every arrive waited for the warp's outstanding global stores, and the tensor core stood idle
//     for 28 % of the product waiting for accumulators (0.5 % with the relaxed arrive; what orders the TMEM reads
//     is tcgen05.wait::ld + tcgen05.fence::before_thread_sync, and no memory is handed over).
// Every wait is bounded as in the other kernels; a CTA that gives up sets the error flag, the other one
// of the pair sees it in its own waits, and both still reach the final cluster barrier.
namespace p2 {
constexpr int BK = 32;
constexpr int UNITS = 6;
constexpr int UNIT_BYTES = 32 * 1024;               // 128 rows of A + 128 rows of B, 128 bytes each
constexpr int BAR_BYTES = 512;
constexpr int SCALE_BYTES = EPI_WARPS * 128 * 4;
constexpr int SMEM_BYTES = UNITS * UNIT_BYTES + 1024 /*alignment slack*/ + BAR_BYTES + SCALE_BYTES;
constexpr int BM2 = 2 * BM;                          // rows of the pair's tile
static_assert(SMEM_BYTES <= 227 * 1024, "unit ring does not fit in shared memory");
}  // namespace p2

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// arrive that orders nothing but itself (the accumulator hand-back: the TMEM reads before it are ordered by
// tcgen05.wait::ld and tcgen05.fence::before_thread_sync, and no memory is handed over)
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_shared_cluster(uint32_t cluster_addr, int v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait on a barrier of this CTA that the other CTA of the pair may arrive at
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* err_flag, int code) {
  for (uint32_t spins = 0;; ++spins) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((spins & 0x3ff) == 0x3ff) {
      if (*((volatile int*)err_flag) != 0) return false;
      if (spins >= SPIN_LIMIT) { atomicCAS(err_flag, 0, code); return false; }
    }
  }
}
// TMA load into this CTA's shared memory whose bytes are counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier (any CTA of the cluster) once every MMA issued so far has completed in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// Instruction descriptor of the pair's product: D = F32, A = B = FP16, K-major, M = 256 over two CTAs, N = 256.
__host__ __device__ constexpr uint32_t idesc_fp16_pair() {
  return (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(p2::BM2 >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 int M, int N, float* __restrict__ C, int64_t ldc, bool vecC, Epi epi,
                 int* __restrict__ err_flag, TileSched ts) {
  using namespace p2;
  extern __shared__ uint8_t smem_raw[];
  // the same offsets in both CTAs: the dynamic shared memory of a kernel starts at the same window offset in each
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + UNITS * UNIT_BYTES;
  constexpr int TQ = 4;
  auto full_bar = [&](uint32_t s) { return bars + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bars + 8u * (UNITS + s); };
  auto acc_full = [&](uint32_t b) { return bars + 8u * (2 * UNITS + b); };
  auto acc_empty = [&](uint32_t b) { return bars + 8u * (2 * UNITS + 2 + b); };
  auto tile_full = [&](uint32_t i) { return bars + 8u * (2 * UNITS + 4 + i); };
  auto tile_empty = [&](uint32_t i) { return bars + 8u * (2 * UNITS + 4 + TQ + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * UNITS + 4 + 2 * TQ);
  const uint32_t tile_q_addr = tmem_slot + 8u;
  uint8_t* generic_base = smem_raw + (base - smem_u32(smem_raw));
  uint8_t* generic_bars = generic_base + UNITS * UNIT_BYTES;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_bars + 8 * (2 * UNITS + 4 + 2 * TQ));
  volatile int* tile_q = reinterpret_cast<volatile int*>(generic_bars + 8 * (2 * UNITS + 4 + 2 * TQ) + 8);
  static_assert(8 * (2 * UNITS + 4 + 2 * TQ) + 8 + 4 * TQ <= BAR_BYTES, "barrier block too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const bool leader = rank == 0;
  const int num_pairs = (int)(gridDim.x >> 1), pair = (int)(blockIdx.x >> 1);
  const int total_tiles = ts.tiles_m * ts.tiles_n * ts.splits;     // tiles of 256 x 256
  int* const tile_counter = err_flag + 32;
  int* const done_counter = err_flag + 33;

  __shared__ int s_abort, s_run;
  if (threadIdx.x == 0) {
    s_abort = *((volatile int*)err_flag);
    for (int s = 0; s < UNITS; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 2 * EPI_WARPS); }
    // queue entries are consumed by the leader's MMA warp and epilogue warps and the other CTA's producer and epilogue warps
    for (int i = 0; i < TQ; ++i) { mbar_init(tile_full(i), 1); mbar_init(tile_empty(i), 2 + 2 * EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();          // barriers of both CTAs initialised before anybody arrives remotely
  // the pair runs or stays out together: both CTAs go by what the leader saw in the error flag (the TMEM
  // allocation below is an operation of the pair)
  if (threadIdx.x == 0) {
    int a;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(a) : "r"(mapa_shared(smem_u32(&s_abort), 0)) : "memory");
    s_run = a == 0;
  }
  __syncthreads();
  const bool run = s_run != 0;
  if (run && warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // TMEM of both CTAs allocated before the leader multiplies into it
  tc_fence_after();
  const uint32_t tmem_base = run ? *tmem_slot_ptr : 0u;

  auto next_tile = [&](uint32_t qi, int role, bool whole_warp) -> int {
    const uint32_t slot = qi % TQ;
    bool got = mbar_wait_cluster(tile_full(slot), (qi / TQ) & 1, err_flag, role);
    if (whole_warp) got = __all_sync(0xffffffffu, got);
    if (!got) return -2;
    const int t = tile_q[slot];
    if (whole_warp) __syncwarp();
    if (lane == 0) mbar_arrive_cluster(mapa_shared(tile_empty(slot), 0));
    return t;
  };
  auto tile_of = [&](int t, int& m0, int& n0, int& z, int& kb0, int& num_kb) {
    const int per_slice = ts.tiles_n * ts.tiles_m;
    z = t / per_slice;
    const int t2 = t - z * per_slice;
    const int p = t2 / (ts.tiles_m * ts.panel_n);
    const int r = t2 - p * ts.tiles_m * ts.panel_n;
    const int w = min(ts.panel_n, ts.tiles_n - p * ts.panel_n);
    m0 = (r / w) * BM2 + (int)rank * BM;            // this CTA's 128 rows of the pair's tile
    n0 = (p * ts.panel_n + r % w) * BN;
    kb0 = z * ts.kb_per_split;
    num_kb = min(ts.total_kb - kb0, ts.kb_per_split);
  };

  if (!run) {
    // nothing: fall through to the final barrier
  } else if (warp == 0) {
    // ------------------------------------------------------------ tile scheduler (leader) + TMA producer (both)
    if (lane == 0) {
      uint32_t g = 0, qi = 0;
      bool ok = true;
      int t = pair;
      while (ok) {
        if (leader) {
          const uint32_t qslot = qi % TQ, qround = qi / TQ;
          if (qround > 0 && !mbar_wait_cluster(tile_empty(qslot), (qround - 1) & 1, err_flag, 5)) break;
          const int pub = t < total_tiles ? t : -1;
          tile_q[qslot] = pub;
          st_shared_cluster(mapa_shared(tile_q_addr + 4u * qslot, 1), pub);
          mbar_arrive(tile_full(qslot));
          mbar_arrive_cluster(mapa_shared(tile_full(qslot), 1));     // release: the entry is visible with the phase
          ++qi;
          if (t >= total_tiles) break;
        } else {
          t = next_tile(qi++, 5, false);
          if (t < 0) break;
        }
        int m0, n0, z, kb0, num_kb;
        tile_of(t, m0, n0, z, kb0, num_kb);
        for (int kb = 0; kb < num_kb && ok; ++kb, ++g) {
          const int x = (kb0 + kb) * BK;
          const uint32_t slot = g % UNITS, round = g / UNITS;
          if (round > 0 && !mbar_wait(empty_bar(slot), (round - 1) & 1, err_flag, 1)) { ok = false; break; }
          const uint32_t st = base + slot * UNIT_BYTES;
          // the leader announces the unit's bytes of both CTAs; both CTAs' loads complete on the leader's barrier
          if (leader) mbar_expect_tx(full_bar(slot), 2 * UNIT_BYTES);
          const uint32_t fb = mapa_shared(full_bar(slot), 0);
          tma_load_2d_pair(st, &map_a, fb, 2 * x, m0);
          tma_load_2d_pair(st + 16 * 1024, &map_b, fb, 2 * x, n0 + (int)rank * (BN / 2));
        }
        if (leader) t = num_pairs + atomicAdd(tile_counter, 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc_q = idesc_fp16_pair();
      uint32_t g = 0, gc = 0, qi = 0;
      bool ok = true;
#ifdef PRAD_GEMM_STALL_PROBE
      long long w_full = 0, w_acc = 0, w_tile = 0;
      const long long t_begin = clock64();
#endif
      while (ok) {
        int t;
        PROBE_WAIT(w_tile, t = next_tile(qi++, 6, false));
        if (t < 0) break;
        int m0, n0, z, kb0, num_kb;
        tile_of(t, m0, n0, z, kb0, num_kb);
        const int num_chunks = (num_kb + ts.chunk_kb - 1) / ts.chunk_kb;
        for (int ch = 0; ch < num_chunks && ok; ++ch, ++gc) {
          const uint32_t buf = gc & 1, use = gc >> 1;
          if (use > 0) {
            PROBE_WAIT(w_acc, ok = mbar_wait_cluster(acc_empty(buf), (use - 1) & 1, err_flag, 4));
            if (!ok) break;
            tc_fence_after();
          }
          const uint32_t d_tmem = tmem_base + buf * (uint32_t)BN;
          const int kb_end = min(num_kb, (ch + 1) * ts.chunk_kb);
          for (int kb = ch * ts.chunk_kb; kb < kb_end && ok; ++kb, ++g) {
            const uint32_t slot = g % UNITS;
            PROBE_WAIT(w_full, ok = mbar_wait(full_bar(slot), (g / UNITS) & 1, err_flag, 2));
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = base + slot * UNIT_BYTES;
            const uint64_t a_0 = kmajor_desc<128>(st), a_1 = a_0 + 4;
            const uint64_t b_0 = kmajor_desc<128>(st + 16 * 1024), b_1 = b_0 + 4;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adv = (uint64_t)((k * 16 * 2) >> 4);
              umma_f16_pair(d_tmem, a_1 + adv, b_0 + adv, idesc_q, !(kb == ch * ts.chunk_kb && k == 0));
              umma_f16_pair(d_tmem, a_0 + adv, b_1 + adv, idesc_q, 1);
              umma_f16_pair(d_tmem, a_0 + adv, b_0 + adv, idesc_q, 1);
            }
            umma_commit_pair(empty_bar(slot));                      // the unit is free again: here ...
            umma_commit_pair(mapa_shared(empty_bar(slot), 1));      // ... and in the other CTA
          }
          umma_commit_pair(acc_full(buf));
          umma_commit_pair(mapa_shared(acc_full(buf), 1));
        }
      }
#ifdef PRAD_GEMM_STALL_PROBE
      if (blockIdx.x == 0)
        printf("pair mma issuer: total %lld cycles, waited for operands %lld, for the accumulator %lld, for tiles %lld (units %u)\n",
               clock64() - t_begin, w_full, w_acc, w_tile, g);
#endif
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int sub = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t gc = 0, qi = 0;
    bool ok = true;
    float4* const sb_slot = reinterpret_cast<float4*>(generic_bars + BAR_BYTES) + (warp - 2) * 32;
    while (ok) {
      const int t = next_tile(qi++, 7, true);
      if (t < 0) break;
      int m0, n0, z, kb0, num_kb;
      tile_of(t, m0, n0, z, kb0, num_kb);
      const int num_chunks = (num_kb + ts.chunk_kb - 1) / ts.chunk_kb;
      float sum[4][32];
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[g][j] = 0.f;
      const int chunk0 = kb0 / ts.chunk_kb;
      const int row_blk = min(m0 + sub * 32 + lane, M - 1);
      float sa_next = 0.f;
      float4 sb_next = make_float4(0.f, 0.f, 0.f, 0.f);
      auto fetch_scales = [&](int ch) {
        sa_next = __ldg(epi.blk_a + (int64_t)(chunk0 + ch) * epi.blk_lda + row_blk);
        sb_next = __ldg(reinterpret_cast<const float4*>(epi.blk_b + (int64_t)(chunk0 + ch) * epi.blk_ldb + n0 + half * 128) + lane);
      };
      fetch_scales(0);
      for (int ch = 0; ch < num_chunks; ++ch, ++gc) {
        const uint32_t buf = gc & 1;
        const float sa = sa_next;
        sb_slot[lane] = sb_next;
        __syncwarp();
        if (ch + 1 < num_chunks) fetch_scales(ch + 1);
        ok = __all_sync(0xffffffffu, mbar_wait(acc_full(buf), (gc >> 1) & 1, err_flag, 3));
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + buf * (uint32_t)BN + (uint32_t)(half * 128);
        const float2 sa2 = make_float2(sa, sa);
        uint32_t v[2][8];
        tmem_ld8(taddr, v[0]);
#pragma unroll
        for (int g = 0; g < 16; ++g) {
          uint32_t (&cur)[8] = v[g & 1];
          tmem_ld_wait8(cur);
          if (g + 1 < 16) tmem_ld8(taddr + (uint32_t)((g + 1) * 8), v[(g + 1) & 1]);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const float4 tq = sb_slot[g * 2 + q];
            float* acc = &sum[g >> 2][(g & 3) * 8 + 4 * q];
            const float2 p01 = __fmul2_rn(make_float2(__uint_as_float(cur[4 * q]), __uint_as_float(cur[4 * q + 1])), sa2);
            const float2 p23 = __fmul2_rn(make_float2(__uint_as_float(cur[4 * q + 2]), __uint_as_float(cur[4 * q + 3])), sa2);
            const float2 r01 = __ffma2_rn(p01, make_float2(tq.x, tq.y), make_float2(acc[0], acc[1]));
            const float2 r23 = __ffma2_rn(p23, make_float2(tq.z, tq.w), make_float2(acc[2], acc[3]));
            acc[0] = r01.x; acc[1] = r01.y; acc[2] = r23.x; acc[3] = r23.y;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive_relaxed(acc_empty(buf));
          else mbar_arrive_cluster_relaxed(mapa_shared(acc_empty(buf), 0));
        }
      }
      if (!ok) break;
      // has another CTA given up?  Asked before the stores and looked at after them: the answer takes a trip to L2
      const int gave_up = *((volatile int*)err_flag);
      float* Ct = C + (int64_t)z * ts.split_stride;
      epilogue_store_warp(sum, lane, m0 + sub * 32, n0 + half * 128, M, N, Ct, ldc, vecC, epi);
      if (gave_up != 0) { ok = false; break; }
    }
  }

  // drain: nobody leaves (or frees TMEM) while the other CTA of the pair may still signal it or multiply into it
  tc_fence_before();
  __syncthreads();
  if (*((volatile int*)err_flag) != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  cluster_sync_all();
  if (run && warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1) == (int)gridDim.x - 1) {
      *((volatile int*)tile_counter) = 0;
      *((volatile int*)done_counter) = 0;
      __threadfence();
    }
  }
}

// ---- operand preparation: hi/lo split (optionally transposing) into K-major scratch -----
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
// src is rows x cols (ld = src_ld); dst_hi/dst_lo are rows x dst_ld with the same orientation
// With xb/lb given (MODE 1) the FP32 `lo` array is not written; xb = bf16(x), lb = bf16(x - hi).
// With b0 given (MODE 2) only the three BF16 pieces b0, xb (= b1), lb (= b2) are written.
__device__ __forceinline__ void bf16_pieces(float x, __nv_bfloat16& p0, __nv_bfloat16& p1, __nv_bfloat16& p2) {
  p0 = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(p0);     // exact
  p1 = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(p1);    // exact
  p2 = __float2bfloat16_rn(r2);
}
__global__ void __launch_bounds__(256)
split_kernel(const float* __restrict__ src, int64_t src_ld, float* __restrict__ hi, float* __restrict__ lo,
             __nv_bfloat16* __restrict__ xb, __nv_bfloat16* __restrict__ lb, __nv_bfloat16* __restrict__ b0,
             int64_t dst_ld, int rows, int cols) {
  const int64_t total = (int64_t)rows * (dst_ld / 4);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool vec = ((src_ld & 3) == 0) && (((uintptr_t)src & 15) == 0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = (int)(i / (dst_ld / 4));
    const int c = (int)(i % (dst_ld / 4)) * 4;
    float x[4];
    if (vec && c + 4 <= cols) {
      float4 v = *reinterpret_cast<const float4*>(src + (int64_t)r * src_ld + c);
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) x[q] = (c + q < cols) ? src[(int64_t)r * src_ld + c + q] : 0.f;
    }
    if (b0) {
      __align__(8) __nv_bfloat16 p0[4];
      __align__(8) __nv_bfloat16 p1[4];
      __align__(8) __nv_bfloat16 p2[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) bf16_pieces(x[q], p0[q], p1[q], p2[q]);
      *reinterpret_cast<uint2*>(b0 + (int64_t)r * dst_ld + c) = *reinterpret_cast<uint2*>(p0);
      *reinterpret_cast<uint2*>(xb + (int64_t)r * dst_ld + c) = *reinterpret_cast<uint2*>(p1);
      *reinterpret_cast<uint2*>(lb + (int64_t)r * dst_ld + c) = *reinterpret_cast<uint2*>(p2);
      continue;
    }
    float h[4], l[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { h[q] = to_tf32(x[q]); l[q] = x[q] - h[q]; }
    *reinterpret_cast<float4*>(hi + (int64_t)r * dst_ld + c) = make_float4(h[0], h[1], h[2], h[3]);
    if (xb) {
      __nv_bfloat162 x01 = __floats2bfloat162_rn(x[0], x[1]), x23 = __floats2bfloat162_rn(x[2], x[3]);
      __nv_bfloat162 l01 = __floats2bfloat162_rn(l[0], l[1]), l23 = __floats2bfloat162_rn(l[2], l[3]);
      uint2 xv = make_uint2(*reinterpret_cast<uint32_t*>(&x01), *reinterpret_cast<uint32_t*>(&x23));
      uint2 lv = make_uint2(*reinterpret_cast<uint32_t*>(&l01), *reinterpret_cast<uint32_t*>(&l23));
      *reinterpret_cast<uint2*>(xb + (int64_t)r * dst_ld + c) = xv;
      *reinterpret_cast<uint2*>(lb + (int64_t)r * dst_ld + c) = lv;
    } else {
      *reinterpret_cast<float4*>(lo + (int64_t)r * dst_ld + c) =
          make_float4(to_tf32(l[0]), to_tf32(l[1]), to_tf32(l[2]), to_tf32(l[3]));
    }
  }
}
// src is rows x cols; dst is cols x dst_ld (transposed), dst_ld >= rows
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ src, int64_t src_ld, float* __restrict__ hi,
                       float* __restrict__ lo, __nv_bfloat16* __restrict__ xb, __nv_bfloat16* __restrict__ lb,
                       __nv_bfloat16* __restrict__ b0, int64_t dst_ld, int rows, int cols) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const int c = blockIdx.x * 32 + tx;
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int r = blockIdx.y * 32 + j;
    tile[j][tx] = (r < rows && c < cols) ? src[(int64_t)r * src_ld + c] : 0.f;
  }
  __syncthreads();
  const int r2 = blockIdx.y * 32 + tx;   // fast index of dst
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int c2 = blockIdx.x * 32 + j;
    if (c2 < cols && r2 < dst_ld) {
      const float x = tile[tx][j];       // zero beyond `rows` (padding columns of dst)
      if (b0) {
        __nv_bfloat16 p0, p1, p2;
        bf16_pieces(x, p0, p1, p2);
        b0[(int64_t)c2 * dst_ld + r2] = p0;
        xb[(int64_t)c2 * dst_ld + r2] = p1;
        lb[(int64_t)c2 * dst_ld + r2] = p2;
        continue;
      }
      const float h = to_tf32(x);
      hi[(int64_t)c2 * dst_ld + r2] = h;
      if (xb) {
        xb[(int64_t)c2 * dst_ld + r2] = __float2bfloat16_rn(x);
        lb[(int64_t)c2 * dst_ld + r2] = __float2bfloat16_rn(x - h);
      } else {
        lo[(int64_t)c2 * dst_ld + r2] = to_tf32(x - h);
      }
    }
  }
}

// C = alpha * (P_0 + P_1 + ... ) + beta * C, slices added in order; P_s are dense M x N.  V = 4: four consecutive
// elements per thread (N, ldc and mn multiples of four, 16-byte aligned pointers).  The loads of eight slices are issued
// before the first of them is added: with 64 slices of a small output (96 x 288 over k = 200 704) the pass was a chain of
// 64 round trips to L2 per thread.
template <int V>
__global__ void __launch_bounds__(256)
splitk_combine_kernel(const float* __restrict__ part, int splits, int64_t mn, int M, int N,
                      float* __restrict__ C, int64_t ldc, float alpha, float beta) {
  constexpr int U = 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * V;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * V; i < mn; i += stride) {
    float acc[V];
    auto fetch = [&](int sl, float (&v)[V]) {
      if (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(part + (int64_t)sl * mn + i);
        v[0] = t.x; v[1 % V] = t.y; v[2 % V] = t.z; v[3 % V] = t.w;
      } else {
        v[0] = part[(int64_t)sl * mn + i];
      }
    };
    fetch(0, acc);
    int sl = 1;
    for (; sl + U <= splits; sl += U) {
      float v[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) fetch(sl + u, v[u]);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = __fadd_rn(acc[q], v[u][q]);
    }
    for (; sl < splits; ++sl) {
      float v[V];
      fetch(sl, v);
#pragma unroll
      for (int q = 0; q < V; ++q) acc[q] = __fadd_rn(acc[q], v[q]);
    }
    const int64_t off = (i / N) * ldc + (i % N);
    float o[V];
#pragma unroll
    for (int q = 0; q < V; ++q) o[q] = __fmul_rn(alpha, acc[q]);
    if (beta != 0.f) {
      float old[V];
      if (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(C + off);
        old[0] = t.x; old[1 % V] = t.y; old[2 % V] = t.z; old[3 % V] = t.w;
      } else {
        old[0] = C[off];
      }
#pragma unroll
      for (int q = 0; q < V; ++q) o[q] = (beta == 1.f) ? __fadd_rn(old[q], o[q]) : fmaf(beta, old[q], o[q]);
    }
    if (V == 4) *reinterpret_cast<float4*>(C + off) = make_float4(o[0], o[1 % V], o[2 % V], o[3 % V]);
    else C[off] = o[0];
  }
}

// ---- host side --------------------------------------------------------------------------
static void launch_splitk_combine(prad_ctx* ctx, const float* part, int splits, int64_t mn, int M, int N, float* C,
                                  int64_t ldc, float alpha, float beta) {
  const bool vec = N % 4 == 0 && ldc % 4 == 0 && (((uintptr_t)C | (uintptr_t)part) & 15) == 0;
  if (vec) {
    const int cg = stream_grid(ctx, mn / 4, 256, 8);
    splitk_combine_kernel<4><<<cg, 256, 0, ctx->stream>>>(part, splits, mn, M, N, C, ldc, alpha, beta);
  } else {
    const int cg = stream_grid(ctx, mn, 256, 8);
    splitk_combine_kernel<1><<<cg, 256, 0, ctx->stream>>>(part, splits, mn, M, N, C, ldc, alpha, beta);
  }
}
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// K-major operand: `rows` rows of `k` floats, row pitch ld floats (ld % 4 == 0)
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int k, int64_t ld, int box_rows, int bk,
                     int elem_bytes = 4, bool fp16 = false) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)box_rows};
  const int row_bytes = bk * elem_bytes;
  CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                           : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : (fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  CUresult r = encode_fn()(map, dt, 2, (void*)ptr, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}



// Operand scratch in K-major form.  MODE 0: hi, lo as FP32.  MODE 1: hi as FP32, xb = bf16(x)
// and lb = bf16(x - hi) as BF16.
struct SplitOperand {
  float* hi = nullptr;
  float* lo = nullptr;
  __nv_bfloat16* xb = nullptr;
  __nv_bfloat16* lb = nullptr;
  __nv_bfloat16* b0 = nullptr;   // MODE 2: pieces are b0, xb (= b1), lb (= b2)
};

// cudaFuncSetAttribute applies to the current device only: once per kernel and device (a second,
// concurrent call for the same pair is harmless)
template <class F>
static cudaError_t reserve_smem(F kernel, int bytes, int device, std::atomic<uint64_t>& done) {
  const uint64_t bit = 1ull << (device & 63);
  if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
  else (void)cudaGetLastError();
  return e;
}

template <class CFG>
static prad_status launch_tf32x3(prad_ctx* ctx, const SplitOperand& a, const SplitOperand& b, int M, int N,
                                 int64_t kp, float* C, int64_t ldc, bool vecC, const Epi& epi) {
  static_assert(CFG::MODE != 3, "packed FP16 operands go through gemm_fp16x3_packed");
  {
    static std::atomic<uint64_t> attr_done{0};
    const cudaError_t attr_err = reserve_smem(gemm_tf32x3_kernel<CFG>, CFG::SMEM_BYTES, ctx->device, attr_done);
    PRAD_REQUIRE(attr_err == cudaSuccess, PRAD_ERR_CUDA, "gemm tf32x3: cannot reserve %d bytes of shared memory: %s",
                 CFG::SMEM_BYTES, cudaGetErrorString(attr_err));
  }
  CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo, ma_x, mb_x;
  bool ok = true;
  if (CFG::MODE == 2) {
    ok = make_map(&ma_hi, a.b0, M, (int)kp, kp, BM, CFG::BK, 2) && make_map(&ma_x, a.xb, M, (int)kp, kp, BM, CFG::BK, 2) &&
         make_map(&ma_lo, a.lb, M, (int)kp, kp, BM, CFG::BK, 2) && make_map(&mb_hi, b.b0, N, (int)kp, kp, BN, CFG::BK, 2) &&
         make_map(&mb_x, b.xb, N, (int)kp, kp, BN, CFG::BK, 2) && make_map(&mb_lo, b.lb, N, (int)kp, kp, BN, CFG::BK, 2);
  } else {
    ok = make_map(&ma_hi, a.hi, M, (int)kp, kp, BM, CFG::BK) && make_map(&mb_hi, b.hi, N, (int)kp, kp, BN, CFG::BK);
  }
  if (CFG::MODE >= 2) {
  } else if (CFG::MODE == 0) {
    ok = ok && make_map(&ma_lo, a.lo, M, (int)kp, kp, BM, CFG::BK) && make_map(&mb_lo, b.lo, N, (int)kp, kp, BN, CFG::BK);
    ma_x = ma_lo;
    mb_x = mb_lo;
  } else {
    ok = ok && make_map(&ma_lo, a.lb, M, (int)kp, kp, BM, CFG::BK, 2) && make_map(&mb_lo, b.lb, N, (int)kp, kp, BN, CFG::BK, 2) &&
         make_map(&ma_x, a.xb, M, (int)kp, kp, BM, CFG::BK, 2) && make_map(&mb_x, b.xb, N, (int)kp, kp, BN, CFG::BK, 2);
  }
  PRAD_REQUIRE(ok, PRAD_ERR_CUDA, "gemm tf32x3: cuTensorMapEncodeTiled failed (M %d N %d K %lld)", M, N, (long long)kp);
  dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(M, BM));
  PRAD_REQUIRE(grid.y <= 65535, PRAD_ERR_UNSUPPORTED, "gemm tf32x3: too many row tiles (%u)", grid.y);
  // Split-K against wave quantisation: with few output tiles and a long k range (the weight
  // gradient dW = A^T dZ) the last wave of CTAs leaves most SMs idle.  Cutting k into `splits`
  // slices multiplies the CTA count; each slice writes its own partial product and a
  // streaming pass adds them in slice order (deterministic), applying alpha and beta.
  const int total_kb = (int)(kp / CFG::BK);
  const int64_t tiles = (int64_t)grid.x * grid.y;
  int splits = 1;
  const bool plain_epi = !epi.bias && !epi.z_out && epi.act == PRAD_ACT_NONE && epi.dact == PRAD_ACT_NONE;
  if (plain_epi && ctx->tc_split_k) {
    auto eff = [&](int sp) {
      const int64_t ctas = tiles * sp;
      return (double)ctas / (double)(ceil_div(ctas, ctx->sm_count) * ctx->sm_count);
    };
    double best = eff(1) * 1.08;   // a split must pay for its extra pass
    for (int sp = 2; sp <= 64; ++sp)
      if (kp / sp >= 1024 && eff(sp) > best * 1.02) { best = eff(sp); splits = sp; }
  }
  // MODE 1 and MODE 3 on the persistent kernel: one CTA per SM walks the tiles (and k-slices)
  constexpr int PMODE = 1;
  const bool persistent = CFG::MODE == 1 && CFG::BK == p1::BK && ctx->tc_persistent;
  if (persistent) {
    static std::atomic<uint64_t> p_done{0};
    const cudaError_t p_err = reserve_smem(gemm_persistent_kernel<PMODE>, p1::SMEM_BYTES, ctx->device, p_done);
    PRAD_REQUIRE(p_err == cudaSuccess, PRAD_ERR_CUDA, "gemm (persistent): cannot reserve %d bytes of shared memory: %s",
                 p1::SMEM_BYTES, cudaGetErrorString(p_err));
  }
  auto launch = [&](int nsplit, int kbps, int64_t stride, float* out, int64_t ldo, bool vec_out, const Epi& ep) {
    if (persistent) {
      // two panels when the column operand (N x k, 4 bytes per element in either scheme's main pieces)
      // would not stay in L2 next to the streaming row operand
      int panel_n = (int)grid.x;
      if (ctx->tc_panel_n > 0) panel_n = ctx->tc_panel_n < (int)grid.x ? ctx->tc_panel_n : (int)grid.x;
      else if ((int64_t)N * kp * 4 > ((int64_t)40 << 20) && grid.x >= 2) panel_n = ((int)grid.x + 1) / 2;
      TileSched ts{(int)grid.y, (int)grid.x, nsplit, kbps, total_kb, ctx->tc_chunk_k / p1::BK, panel_n, stride};
      const int64_t total = tiles * nsplit;
      const int64_t sms = ctx->sm_count - ctx->tc_reserve_sms;
      const unsigned ctas = (unsigned)(total < sms ? total : sms);
      gemm_persistent_kernel<PMODE><<<ctas, THREADS, p1::SMEM_BYTES, ctx->stream>>>(
          ma_hi, ma_x, ma_lo, mb_hi, mb_x, mb_lo, M, N, out, ldo, vec_out, ep, ctx->tc_err, ts);
    } else {
      dim3 g3 = grid;
      g3.z = (unsigned)nsplit;
      gemm_tf32x3_kernel<CFG><<<g3, THREADS, CFG::SMEM_BYTES, ctx->stream>>>(
          ma_hi, ma_lo, mb_hi, mb_lo, ma_x, mb_x, M, N, (int)kp, out, ldo, vec_out, ep, ctx->tc_err, kbps, stride);
    }
  };
  if (splits == 1) {
    launch(1, total_kb, 0, C, ldc, vecC, epi);
    PRAD_LAUNCHED(ctx);
  } else {
    const int64_t mn = (int64_t)M * N;
    prad_status st = ensure_stage(ctx, (size_t)splits * mn * sizeof(float));
    if (st) return st;
    float* part = (float*)ctx->stage;
    Epi raw = epi;
    raw.alpha = 1.f;
    raw.beta = 0.f;
    // k-blocks per slice rounded up to whole accumulation chunks, so slices start on chunk boundaries
    int kbps = (int)ceil_div(ceil_div(total_kb, splits), CFG::CHUNK_KB) * CFG::CHUNK_KB;
    splits = (int)ceil_div(total_kb, kbps);   // no empty slice
    // (the slices are dense M x N blocks: their rows are whole 16-byte vectors only when N is a multiple of four)
    launch(splits, kbps, mn, part, N, N % 4 == 0, raw);
    PRAD_LAUNCHED(ctx);
    launch_splitk_combine(ctx, part, splits, mn, M, N, C, ldc, epi.alpha, epi.beta);
    PRAD_LAUNCHED(ctx);
  }
  ctx->tc_pending_check = true;
  return PRAD_OK;
}

// writes the split form of one operand; `transposed` = the caller's matrix has k as its slow index
static prad_status split_operand(prad_ctx* ctx, const float* src, int64_t ld, bool transposed, int rows, int K,
                                 int64_t kp, const SplitOperand& o) {
  if (!transposed) {
    int grid = stream_grid(ctx, (int64_t)rows * (kp / 4), 256, 8);
    split_kernel<<<grid, 256, 0, ctx->stream>>>(src, ld, o.hi, o.lo, o.xb, o.lb, o.b0, kp, rows, K);
  } else {
    dim3 grid((unsigned)ceil_div(rows, 32), (unsigned)ceil_div(kp, 32));
    split_transpose_kernel<<<grid, 256, 0, ctx->stream>>>(src, ld, o.hi, o.lo, o.xb, o.lb, o.b0, kp, K, rows);
  }
  PRAD_LAUNCHED(ctx);
  return PRAD_OK;
}

// The persistent kernel on two packed FP16 operands (pack_fp16.cuh): C = alpha * A B^T + beta * C (+ bias).
static prad_status launch_fp16x3(prad_ctx* ctx, const PackedForm& a, const PackedForm& b, float* C, int64_t ldc,
                                 float alpha, float beta, const float* bias) {
  const int M = a.rows, N = b.rows;
  const int64_t kp = a.kp;
  PRAD_REQUIRE(encode_fn() != nullptr, PRAD_ERR_UNSUPPORTED, "gemm (tensor core): the driver lacks cuTensorMapEncodeTiled");
  PRAD_REQUIRE(a.kp == b.kp && a.chunk == b.chunk && a.chunk % p1::BK == 0, PRAD_ERR_SHAPE,
               "gemm (tensor core): packed operands disagree in k (%lld, %lld) or block length (%d, %d)",
               (long long)a.kp, (long long)b.kp, a.chunk, b.chunk);
  CUtensorMap ma, mb;
  // interleaved pieces: a row is 2 kp halves, a k-group of 32 is one 128-byte box row (h0 | h1)
  const bool ok = make_map(&ma, a.h, M, (int)(2 * kp), a.pitch, BM, 2 * p1::BK, 2, true) &&
                  make_map(&mb, b.h, N, (int)(2 * kp), b.pitch, BN, 2 * p1::BK, 2, true);
  PRAD_REQUIRE(ok, PRAD_ERR_CUDA, "gemm (tensor core): cuTensorMapEncodeTiled failed (M %d N %d K %lld)", M, N, (long long)kp);
  static std::atomic<uint64_t> p_done{0};
  const cudaError_t p_err = reserve_smem(gemm_persistent_kernel<3>, p1::SMEM_BYTES, ctx->device, p_done);
  PRAD_REQUIRE(p_err == cudaSuccess, PRAD_ERR_CUDA, "gemm (persistent): cannot reserve %d bytes of shared memory: %s",
               p1::SMEM_BYTES, cudaGetErrorString(p_err));
  const int tiles_m = (int)ceil_div(M, BM), tiles_n = (int)ceil_div(N, BN);
  const int64_t tiles = (int64_t)tiles_m * tiles_n;
  const int total_kb = (int)(kp / p1::BK), chunk_kb = a.chunk / p1::BK;
  // CTA pairs (256-row tiles over two SMs) when the output has at least two tile rows and the option allows
  const int tiles_m2 = (int)ceil_div(M, p2::BM2);
  // (not for k below 1024 with fewer than 1024 columns: a pair halves the shared-memory traffic of the column operand,
  // which long k loops and wide outputs feel, while its tile transitions cost more -- 200704 x 96 outputs over k = 96 ..
  // 384 take 52 .. 90 us on single CTAs and 61 .. 105 us on pairs; 65536 x 4096 over k = 512 takes 733 and 721 us,
  // 65536 x 1024 over k = 512 about 200 us either way)
  const bool pair = ctx->tc_pair != 0 && M > BM && (kp >= 1024 || N >= 1024 || ctx->tc_pair == 2) &&
                    ctx->sm_count - ctx->tc_reserve_sms >= 2;
  CUtensorMap mb_half;
  if (pair) {
    PRAD_REQUIRE(make_map(&mb_half, b.h, N, (int)(2 * kp), b.pitch, BN / 2, 2 * p1::BK, 2, true), PRAD_ERR_CUDA,
                 "gemm (tensor core): cuTensorMapEncodeTiled failed for the half column tile (N %d K %lld)", N, (long long)kp);
    static std::atomic<uint64_t> pair_done{0};
    const cudaError_t q_err = reserve_smem(gemm_pair_kernel, p2::SMEM_BYTES, ctx->device, pair_done);
    PRAD_REQUIRE(q_err == cudaSuccess, PRAD_ERR_CUDA, "gemm (CTA pairs): cannot reserve %d bytes of shared memory: %s",
                 p2::SMEM_BYTES, cudaGetErrorString(q_err));
  }
  // Split-K against wave quantisation (see launch_tf32x3); slices start on block boundaries
  int splits = 1;
  if (!bias && ctx->tc_split_k) {
    auto eff = [&](int sp) {
      const int64_t ctas = tiles * sp;
      return (double)ctas / (double)(ceil_div(ctas, ctx->sm_count) * ctx->sm_count);
    };
    double best = eff(1) * 1.08;   // a split must pay for its extra pass
    for (int sp = 2; sp <= 64; ++sp)
      if (kp / sp >= 1024 && eff(sp) > best * 1.02) { best = eff(sp); splits = sp; }
  }
  const bool vecC = (((uintptr_t)C & 15) == 0) && (ldc % 4 == 0);
  Epi epi{bias, nullptr, 0, 0, nullptr, 0.f, alpha, beta, nullptr, nullptr, a.blk, b.blk, a.rows_ld, b.rows_ld};
  auto launch = [&](int nsplit, int kbps, int64_t stride, float* out, int64_t ldo, bool vec_out, const Epi& ep) {
    int panel_n = tiles_n;
    if (ctx->tc_panel_n > 0) panel_n = ctx->tc_panel_n < tiles_n ? ctx->tc_panel_n : tiles_n;
    else if ((int64_t)N * kp * 4 > ((int64_t)40 << 20) && tiles_n >= 2) panel_n = (tiles_n + 1) / 2;
    const int64_t sms = ctx->sm_count - ctx->tc_reserve_sms;
    if (pair) {
      TileSched ts{tiles_m2, tiles_n, nsplit, kbps, total_kb, chunk_kb, panel_n, stride};
      const int64_t total = (int64_t)tiles_m2 * tiles_n * nsplit;
      const int64_t pairs = sms / 2;
      const unsigned ctas = 2u * (unsigned)(total < pairs ? total : pairs);
      gemm_pair_kernel<<<ctas, THREADS, p2::SMEM_BYTES, ctx->stream>>>(ma, mb_half, M, N, out, ldo, vec_out, ep, ctx->tc_err, ts);
      return;
    }
    TileSched ts{tiles_m, tiles_n, nsplit, kbps, total_kb, chunk_kb, panel_n, stride, ctx->tc_prefetch};
    const int64_t total = tiles * nsplit;
    const unsigned ctas = (unsigned)(total < sms ? total : sms);
    gemm_persistent_kernel<3><<<ctas, THREADS, p1::SMEM_BYTES, ctx->stream>>>(ma, ma, ma, mb, mb, mb, M, N, out, ldo, vec_out,
                                                                              ep, ctx->tc_err, ts);
  };
  if (splits == 1) {
    launch(1, total_kb, 0, C, ldc, vecC, epi);
    PRAD_LAUNCHED(ctx);
  } else {
    const int64_t mn = (int64_t)M * N;
    prad_status st = ensure_stage(ctx, (size_t)splits * mn * sizeof(float));
    if (st) return st;
    float* part = (float*)ctx->stage;
    Epi raw = epi;
    raw.alpha = 1.f;
    raw.beta = 0.f;
    int kbps = (int)ceil_div(ceil_div(total_kb, splits), chunk_kb) * chunk_kb;
    splits = (int)ceil_div(total_kb, kbps);   // no empty slice
    // (the slices are dense M x N blocks: their rows are whole 16-byte vectors only when N is a multiple of four)
    launch(splits, kbps, mn, part, N, N % 4 == 0, raw);
    PRAD_LAUNCHED(ctx);
    launch_splitk_combine(ctx, part, splits, mn, M, N, C, ldc, alpha, beta);
    PRAD_LAUNCHED(ctx);
  }
  ctx->tc_pending_check = true;
  return PRAD_OK;
}

}  // namespace tc

prad_status gemm_fp16x3_packed(prad_ctx* ctx, const PackedForm& a, const PackedForm& b, float alpha, float beta,
                               float* C, int64_t ldc, const float* bias) {
  return tc::launch_fp16x3(ctx, a, b, C, ldc, alpha, beta, bias);
}

prad_status gemm_tf32x3(prad_ctx* ctx, bool tA, bool tB, int M, int N, int K, double alpha,
                        const void* A, int lda, const void* B, int ldb, double beta, void* C,
                        int ldc, int batch, int64_t sA, int64_t sB, int64_t sC,
                        const GemmEpilogue& e, bool probe_only) {
  using namespace tc;
  (void)sA; (void)sB; (void)sC;
  // shapes this kernel is meant for; everything else stays on the SIMT variant
  const bool forced = ctx->gemm_f32 == GemmF32::Tf32x3 || ctx->gemm_f32 == GemmF32::Tf32B16 ||
                      ctx->gemm_f32 == GemmF32::Bf16x3 || ctx->gemm_f32 == GemmF32::Fp16x3;
  // large products; a short M or N only wastes part of the 128 x 256 tile (TMA zero-fills it),
  // which still beats ten CTAs walking a 200 000-long k range one after the other
  const bool big = (int64_t)M * N * K >= ((int64_t)1 << 27) && M >= 64 && N >= 64 && K >= KPAD;
  // (an activation or pre-activation copy on a strided output would need a strided elementwise pass)
  const bool strided_act = ldc != N && (e.act != PRAD_ACT_NONE || e.dact != PRAD_ACT_NONE || e.z_out);
  if (batch != 1 || K < 1 || !(big || forced) || strided_act || encode_fn() == nullptr) {
    if (probe_only || !forced) return PRAD_ERR_UNSUPPORTED;
    set_error("gemm tf32x3: unsupported shape (batch %d) or driver without cuTensorMapEncodeTiled", batch);
    return PRAD_ERR_UNSUPPORTED;
  }
  if (probe_only) return PRAD_OK;
  // Activations (and the pre-activation copy) run as separate streaming passes.  Measured on the
  // 65536 x 4096 x 4096 products: the epilogue warps hold the whole 128-column row slice in
  // registers, so an activation's loads and transcendental chains run with next to no latency
  // hiding and stall the tensor pipe behind them -- 9.1 ms with GELU and the pre-activation copy
  // fused, 7.6 ms with the GELU derivative fused, against 5.0 ms plain plus 0.4 - 0.5 ms for the
  // HBM-bound elementwise kernel.  The tensor-core epilogues therefore carry no activation code.
  const bool has_act = e.act != PRAD_ACT_NONE, has_dact = e.dact != PRAD_ACT_NONE;
  if (has_act || has_dact || e.z_out) {
    GemmEpilogue plain = e;
    plain.act = PRAD_ACT_NONE;
    plain.dact = PRAD_ACT_NONE;
    plain.saved = nullptr;
    plain.z_out = nullptr;
    const int64_t n = (int64_t)M * N;
    // the pre-activation lands where the caller keeps it; beta needs the old C, so then it is copied
    const bool direct = has_act && e.z_out && beta == 0.0;
    void* pre = direct ? e.z_out : C;
    prad_status st = gemm_tf32x3(ctx, tA, tB, M, N, K, alpha, A, lda, B, ldb, beta, pre, ldc, batch, sA, sB, sC, plain,
                                 false);
    if (st) return st;
    if (e.z_out && !direct) PRAD_CUDA(cudaMemcpyAsync(e.z_out, C, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    if (has_act) st = prad_act_forward(ctx, PRAD_F32, e.act, pre, C, n, e.act_alpha);
    if (st) return st;
    if (has_dact) st = prad_act_backward(ctx, PRAD_F32, e.dact, e.saved, C, C, n, e.act_alpha);
    return st;
  }
  const int mode = ctx->gemm_f32 == GemmF32::Tf32x3 ? 0
                   : ctx->gemm_f32 == GemmF32::Tf32B16 ? 1
                   : ctx->gemm_f32 == GemmF32::Bf16x3 ? 2
                   : ctx->gemm_f32 == GemmF32::Fp16x3 ? 3 : ctx->tc_auto_mode;
  if (mode == 3) {
    // both operands are packed into scratch (pieces, then block exponents), each in one pass
    const int chunk = (ctx->tc_chunk_k_set && ctx->tc_chunk_k >= 256) ? 256 : 128;   // 128: the packing kernel's fast tile
    PackedForm fa = packed_form_shape(M, K, chunk), fb = packed_form_shape(N, K, chunk);
    auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t need = al(fa.h_bytes()) + al(fb.h_bytes()) + al(fa.blk_bytes()) + al(fb.blk_bytes());
    prad_status s3 = ensure_workspace(ctx, need);
    if (s3) return s3;
    char* w = (char*)ctx->ws;
    fa.h = (__half*)w; w += al(fa.h_bytes());
    fb.h = (__half*)w; w += al(fb.h_bytes());
    fa.blk = (float*)w; w += al(fa.blk_bytes());
    fb.blk = (float*)w;
    // exponents of rows beyond the matrices are read by the last tiles: they must be valid (zero)
    PRAD_CUDA(cudaMemsetAsync(fa.blk, 0, al(fa.blk_bytes()) + al(fb.blk_bytes()), ctx->stream));
    PackSource sa, sb;
    sa.x = (const float*)A; sa.ld = lda;
    sb.x = (const float*)B; sb.ld = ldb;
    // op(A) is M x K: memory is M x K unless tA (then K x M, packed by columns).  op(B) is K x N and the
    // kernel wants N x K: memory already is that when tB, otherwise it is packed by columns.
    s3 = tA ? pack_fp16(ctx, sa, K, M, nullptr, &fa) : pack_fp16(ctx, sa, M, K, &fa, nullptr);
    if (s3) return s3;
    s3 = tB ? pack_fp16(ctx, sb, N, K, &fb, nullptr) : pack_fp16(ctx, sb, K, N, nullptr, &fb);
    if (s3) return s3;
    return launch_fp16x3(ctx, fa, fb, (float*)C, ldc, (float)alpha, (float)beta, (const float*)e.bias);
  }

  // scratch: both operands K-major with pitch kp, 8 bytes per element in either mode
  const int64_t kp = ceil_div(K, KPAD) * KPAD;
  const size_t a_elems = (size_t)M * kp, b_elems = (size_t)N * kp;
  const size_t need = 2 * (a_elems + b_elems) * sizeof(float);
  prad_status s = ensure_workspace(ctx, need);
  if (s) return s;
  SplitOperand a, b;
  a.hi = (float*)ctx->ws;
  b.hi = a.hi + 2 * a_elems;
  if (mode == 2) {
    a.b0 = (__nv_bfloat16*)a.hi;
    a.xb = a.b0 + a_elems;
    a.lb = a.xb + a_elems;
    b.b0 = (__nv_bfloat16*)b.hi;
    b.xb = b.b0 + b_elems;
    b.lb = b.xb + b_elems;
  } else if (mode == 0) {
    a.lo = a.hi + a_elems;
    b.lo = b.hi + b_elems;
  } else {
    a.xb = (__nv_bfloat16*)(a.hi + a_elems);
    a.lb = a.xb + a_elems;
    b.xb = (__nv_bfloat16*)(b.hi + b_elems);
    b.lb = b.xb + b_elems;
  }
  // op(A) is M x K: memory is M x K (k contiguous) unless tA.  op(B) is K x N and the kernel
  // wants its transpose N x K (k contiguous): memory already is that when tB.
  s = split_operand(ctx, (const float*)A, lda, tA, M, K, kp, a);
  if (s) return s;
  s = split_operand(ctx, (const float*)B, ldb, !tB, N, K, kp, b);
  if (s) return s;

  Epi epi{(const float*)e.bias, (float*)e.z_out, (int)e.act, (int)e.dact, (const float*)e.saved,
          (float)e.act_alpha, (float)alpha, (float)beta, nullptr, nullptr};
  const bool vecC = (((uintptr_t)C & 15) == 0) && (ldc % 4 == 0) &&
                    (!e.saved || ((uintptr_t)e.saved & 15) == 0);
  float* Cf = (float*)C;
  if (mode == 2) return launch_tf32x3<Cfg<32, 3, 2>>(ctx, a, b, M, N, kp, Cf, ldc, vecC, epi);
  // MODE 1 always runs 32-float k-blocks: with 16 its BF16 tiles would have 32-byte rows, and
  // 32-byte TMA boxes / 32-byte swizzle measured 30 % slower
  if (mode == 1) return launch_tf32x3<Cfg<32, 2, 1>>(ctx, a, b, M, N, kp, Cf, ldc, vecC, epi);
  switch (ctx->tc_variant) {
    case 1: return launch_tf32x3<Cfg<32, 2>>(ctx, a, b, M, N, kp, Cf, ldc, vecC, epi);
    case 2: return launch_tf32x3<Cfg<8, 8>>(ctx, a, b, M, N, kp, Cf, ldc, vecC, epi);
    default: return launch_tf32x3<Cfg<16, 4>>(ctx, a, b, M, N, kp, Cf, ldc, vecC, epi);
  }
}

// ---- self-test of the give-up path ----------------------------------------------------------
// One CTA initialises an mbarrier that nothing will ever arrive on and waits for it with the same
// polling loop as the GEMM kernels, but with a caller-chosen limit of a few polls: the wait runs out,
// the kernel raises the give-up flag (role 9) and returns normally.  Nothing faults and nothing
// hangs; the host then sees PRAD_ERR_TIMEOUT at its next prad_sync, exactly as after a real give-up.
namespace tc {
__global__ void bounded_wait_probe_kernel(int* __restrict__ err_flag, uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool done = false;
    for (uint32_t spins = 0; spins < polls && !done; ++spins) done = mbar_try_wait(b, 0);
    if (!done) atomicCAS(err_flag, 0, 9);
  }
}
}  // namespace tc

extern "C" prad_status prad_selftest_bounded_wait(prad_ctx* ctx, int polls) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(polls >= 1 && polls <= (1 << 20), PRAD_ERR_INVALID, "prad_selftest_bounded_wait: polls must be in [1, 2^20]");
  tc::bounded_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->tc_err, (uint32_t)polls);
  PRAD_LAUNCHED(ctx);
  ctx->tc_pending_check = true;
  return PRAD_OK;
}

// Reads the give-up flag of the most recent tensor-core GEMMs (called by prad_sync).
prad_status gemm_tf32x3_check(prad_ctx* ctx) {
  if (!ctx->tc_pending_check || !ctx->tc_err) return PRAD_OK;
  ctx->tc_pending_check = false;
  int flag = 0;
  PRAD_CUDA(cudaMemcpyAsync(&flag, ctx->tc_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  if (flag != 0) PRAD_CUDA(cudaMemsetAsync(ctx->tc_err, 0, 256, ctx->stream));   // flag and tile counters
  PRAD_REQUIRE(flag == 0, PRAD_ERR_TIMEOUT,
               "gemm (tensor core): a bounded wait ran out inside the kernel (role %d: 1 producer, 2 MMA, 3 epilogue, "
               "4 accumulator hand-back, 5-7 tile queue, 9 self-test); "
               "the results of that product are invalid", flag);
  return PRAD_OK;
}

}  // namespace prad
