// Device-side building blocks of the W4A16 GEMV (w4_gemv.cu): the int4 -> bf16 unpack feeding
// mma.sync, mbarrier / bulk-copy wrappers for the per-warp weight rings, and the tile epilogues.
//
// Wire format (python/qengine/quant.py:1-30 of the reference): a matrix is a stream of 1 KB units,
// unit u = tile * G + g = int4 codes of 16 rows x 128 k, stored as two 512-byte chunks of 32 lanes
// x 16 bytes. Lane l = 4 r + t of chunk c owns rows r, r + 8 and k = 64 c + 16 t + 0..15; word s
// of its 16 bytes holds k0 = 64 c + 16 t + 4 s .. k0 + 3 for both rows, nibble j = row
// r + 8 (j & 1), k0 + 2 ((j >> 1) & 1) + (j >> 2). fp16 scales: 16 per unit (one per row).
#pragma once
#include "../../include/qengine_b200.h"
#include "common.cuh"

namespace qb {
namespace w4 {

// ---- int4 -> bf16 ------------------------------------------------------------------------------
// (w >> 4 j) & 0x000F000F picks nibbles j and j + 4 of a word: the same row, two consecutive k.
// OR-ing 0x4300 into each half makes the bf16 number 128 + code (the code lands in the low
// mantissa bits of a number whose ulp is 1); subtracting 136 leaves code - 8 exactly. Four such
// registers of one word are exactly the A fragment of mma.m16n8k16 for rows (r, r + 8) and the
// four k of the word, in a k order that the B fragment (the x values of the same k) mirrors.
__device__ __forceinline__ uint32_t nib2bf16(uint32_t w) {
  uint32_t v;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(v) : "r"(w));  // (w & m) | magic
  asm("sub.rn.bf16x2 %0, %0, %1;" : "+r"(v) : "r"(0x43084308u));
  return v;
}

// A fragment of one packed word: rows (r, r + 8) x the word's four k.
struct AFrag {
  uint32_t a0, a1, a2, a3;
};
__device__ __forceinline__ AFrag unpack_word(uint32_t word) {
  return AFrag{nib2bf16(word), nib2bf16(word >> 4), nib2bf16(word >> 8), nib2bf16(word >> 12)};
}
// c = A(word) * B(xa, xb): first product of a unit (no accumulator to read).
__device__ __forceinline__ void mma_first(float (&c)[4], uint32_t word, uint32_t xa, uint32_t xb) {
  const AFrag f = unpack_word(word);
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(f.a0), "r"(f.a1), "r"(f.a2), "r"(f.a3), "r"(xa), "r"(xb), "f"(0.f));
}
// c += A(word) * B(xa, xb): 16 rows x 4 k of weights times 4 k x 8 activation rows.
__device__ __forceinline__ void mma_word(float (&c)[4], uint32_t word, uint32_t xa, uint32_t xb) {
  const AFrag f = unpack_word(word);
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(f.a0), "r"(f.a1), "r"(f.a2), "r"(f.a3), "r"(xa), "r"(xb));
}

// ---- int4 -> fp16 (activations held as fp16) ------------------------------------------------------
// fp16 has ten mantissa bits: the nibbles at bits 0..3 AND at bits 4..7 of a half-word both sit
// inside the mantissa of 0x6400 | bits (= 1024 + u, resp. 1024 + 16 u). The first becomes u - 8
// by subtracting 1032, the second by one fused multiply-add, (1024 + 16 u) / 16 - 72. Only the
// upper byte needs a shift: one SHF per word instead of three on the half-rate ALU pipe, the
// busiest unit of the kernel (bf16 has seven mantissa bits, where this does not work).
__device__ __forceinline__ uint32_t nib2f16_lo(uint32_t w) {
  uint32_t v;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(v) : "r"(w));
  asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(v) : "r"(0x64086408u));  // - 1032
  return v;
}
__device__ __forceinline__ uint32_t nib2f16_hi(uint32_t w) {
  uint32_t v;
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(v) : "r"(w));
  asm("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(v) : "r"(0x2C002C00u), "r"(0xD480D480u));  // * 2^-4 - 72
  return v;
}
__device__ __forceinline__ AFrag unpack_word_f16(uint32_t word) {
  const uint32_t up = word >> 8;
  return AFrag{nib2f16_lo(word), nib2f16_hi(word), nib2f16_lo(up), nib2f16_hi(up)};
}
__device__ __forceinline__ void mma_first_f16(float (&c)[4], uint32_t word, uint32_t xa, uint32_t xb) {
  const AFrag f = unpack_word_f16(word);
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(f.a0), "r"(f.a1), "r"(f.a2), "r"(f.a3), "r"(xa), "r"(xb), "f"(0.f));
}
__device__ __forceinline__ void mma_word_f16(float (&c)[4], uint32_t word, uint32_t xa, uint32_t xb) {
  const AFrag f = unpack_word_f16(word);
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(f.a0), "r"(f.a1), "r"(f.a2), "r"(f.a3), "r"(xa), "r"(xb));
}

// Operands of one unit for one lane: 2 x 16 B of codes, 2 scales (rows r, r + 8), 32 x values.
struct UnitOps {
  uint4 w0, w1;
  uint4 x0, x1, x2, x3;
  uint32_t s_lo, s_hi;  // raw fp16 bits
};

// acc += scale * (codes - 8) . x for one unit: eight tensor-core products into one fp32 tile, the
// group scale applied once (exact products, fp32 accumulation: the reference's arithmetic,
// csrc/gemv_w4.cu:6-9). The unpack of word i + 1 does not depend on product i, so one accumulator
// chain keeps the pipes busy.
__device__ __forceinline__ void unit_fma(float (&acc)[4], const UnitOps& o) {
  float c[4];
  mma_first(c, o.w0.x, o.x0.x, o.x0.y);
  mma_word(c, o.w0.y, o.x0.z, o.x0.w);
  mma_word(c, o.w0.z, o.x1.x, o.x1.y);
  mma_word(c, o.w0.w, o.x1.z, o.x1.w);
  mma_word(c, o.w1.x, o.x2.x, o.x2.y);
  mma_word(c, o.w1.y, o.x2.z, o.x2.w);
  mma_word(c, o.w1.z, o.x3.x, o.x3.y);
  mma_word(c, o.w1.w, o.x3.z, o.x3.w);
  const float lo = __half2float(__ushort_as_half((unsigned short)o.s_lo));
  const float hi = __half2float(__ushort_as_half((unsigned short)o.s_hi));
  acc[0] = fmaf(lo, c[0], acc[0]);
  acc[1] = fmaf(lo, c[1], acc[1]);
  acc[2] = fmaf(hi, c[2], acc[2]);
  acc[3] = fmaf(hi, c[3], acc[3]);
}

// The same with fp16 activations: the products are exact either way (4-bit code times an 8-bit
// significand), so for activations that fp16 holds exactly the sums have the same bits.
__device__ __forceinline__ void unit_fma_f16(float (&acc)[4], const UnitOps& o) {
  float c[4];
  mma_first_f16(c, o.w0.x, o.x0.x, o.x0.y);
  mma_word_f16(c, o.w0.y, o.x0.z, o.x0.w);
  mma_word_f16(c, o.w0.z, o.x1.x, o.x1.y);
  mma_word_f16(c, o.w0.w, o.x1.z, o.x1.w);
  mma_word_f16(c, o.w1.x, o.x2.x, o.x2.y);
  mma_word_f16(c, o.w1.y, o.x2.z, o.x2.w);
  mma_word_f16(c, o.w1.z, o.x3.x, o.x3.y);
  mma_word_f16(c, o.w1.w, o.x3.z, o.x3.w);
  const float lo = __half2float(__ushort_as_half((unsigned short)o.s_lo));
  const float hi = __half2float(__ushort_as_half((unsigned short)o.s_hi));
  acc[0] = fmaf(lo, c[0], acc[0]);
  acc[1] = fmaf(lo, c[1], acc[1]);
  acc[2] = fmaf(hi, c[2], acc[2]);
  acc[3] = fmaf(hi, c[3], acc[3]);
}

// ---- mbarrier + bulk copy (TMA engine, untiled form) ---------------------------------------------
__device__ __forceinline__ uint32_t sa(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void bar_init(uint64_t* b, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sa(b)), "r"(arrivals));
}
__device__ __forceinline__ void bar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sa(b)), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity: false when the limit ran out (the caller records an error).
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity, int limit) {
  const uint32_t addr = sa(b);
  for (int it = 0; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`. Both addresses and the
// size are multiples of 16 bytes by construction (units are 1024 B, scale rows 32 B).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   sa(dst)), "l"(src), "r"(bytes), "r"(sa(bar))
               : "memory");
}
__device__ __forceinline__ void async_proxy_fence() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- epilogues ---------------------------------------------------------------------------------
struct OutDesc {
  void* out;
  long ldo;
  int M, N;
  int epi;      // QE_EPI_*
  int out_f32;  // plain epilogue only: unrounded fp32 sums (partial results of a K-split matrix)
};

__device__ __forceinline__ float silu_fast(float v) { return v / (1.0f + __expf(-v)); }

// A finished 16 x 8 tile in mma C layout: lane (r = lane / 4, t = lane % 4) holds rows r, r + 8
// of activation rows 2 t, 2 t + 1. With the SwiGLU epilogue rows 0..7 of a tile are gate rows and
// rows 8..15 the matching up rows (quantize_w4_gate_up, python/qengine/quant.py:114-125), so one
// lane holds both halves of its outputs: bf16(silu(gate) * up), fp32 math, one rounding
// (reference epilogue csrc/gemv_w4.cu:188-193).
// `mask` bit k set = write f[k] (plain epilogues only; SwiGLU needs all four values of a lane).
__device__ __forceinline__ void tile_out(const OutDesc& d, int tile, const float (&f)[4], int lane,
                                         unsigned mask = 0xFu) {
  const int r = lane >> 2, n0 = 2 * (lane & 3);
  if (d.epi == QE_EPI_SWIGLU) {
    const int j = tile * 8 + r;
    if (j >= d.M) return;
    bf16* o = static_cast<bf16*>(d.out);
    if (n0 < d.N) o[(long)n0 * d.ldo + j] = tobf16(silu_fast(f[0]) * f[2]);
    if (n0 + 1 < d.N) o[(long)(n0 + 1) * d.ldo + j] = tobf16(silu_fast(f[1]) * f[3]);
    return;
  }
  const int m0 = tile * 16 + r, m1 = m0 + 8;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int n = n0 + c;
    if (n >= d.N) continue;
    const bool w0 = m0 < d.M && (mask >> c & 1u), w1 = m1 < d.M && (mask >> (2 + c) & 1u);
    if (d.out_f32) {
      float* o = static_cast<float*>(d.out) + (long)n * d.ldo;
      if (w0) o[m0] = f[c];
      if (w1) o[m1] = f[2 + c];
    } else {
      bf16* o = static_cast<bf16*>(d.out) + (long)n * d.ldo;
      if (w0) o[m0] = tobf16(f[c]);
      if (w1) o[m1] = tobf16(f[2 + c]);
    }
  }
}

// Equal contiguous shares of `total` items among `parts` owners; the first total % parts owners
// hold one item more.
__device__ __host__ __forceinline__ int share_begin(int total, int parts, int i) {
  const int per = total / parts, rem = total - per * parts;
  return i * per + (i < rem ? i : rem);
}
__device__ __host__ __forceinline__ int share_owner(int total, int parts, int item) {
  const int per = total / parts, rem = total - per * parts;
  const int big = rem * (per + 1);
  return item < big ? item / (per + 1) : rem + (item - big) / per;
}

}  // namespace w4
}  // namespace qb
