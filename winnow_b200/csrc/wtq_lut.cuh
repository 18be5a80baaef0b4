// Device helpers shared by the kernels that turn packed codes into fp16 tensor-
// core operands through per-lane shared-memory tables (the page scan of
// wtq_decode_mma.cu and the tensor-core dequantisation of wtq_dequant.cu).
//
// Table layout: word [index][side][lane] at shared address kLutAddr = 0x10000,
// i.e. 0x10000 | index << 8 | side << 7 | lane << 2: every lane reads its own
// bank (no conflicts whatever the indices) and the address needs no addition.
//   4-bit widths: index = a packed byte, entry = half2 {c[lo nibble], c[hi nibble]}
//   6/8-bit:      index = a code,        entry = half2 {c, c}
#pragma once

#include "wtq_common.cuh"

namespace wtq {
namespace mma {

constexpr uint32_t kLutAddr = 0x10000;                 // shared address of the tables
constexpr int lut_entries(int bw) { return bw == 4 ? 256 : (1 << bw); }

// Word e of the tables for key/value widths (bw_k, bw_v) and codebooks (ck, cv).
__device__ __forceinline__ uint32_t lut_word(int e, int bw_k, int bw_v, const float *ck,
                                             const float *cv) {
  const int index = e >> 6, side = (e >> 5) & 1;
  const int bw = side ? bw_v : bw_k;
  const float *cent = side ? cv : ck;
  __half2 h = __floats2half2_rn(0.f, 0.f);
  if (bw == 4) h = __floats2half2_rn(__ldg(cent + (index & 15)), __ldg(cent + (index >> 4)));
  else if (index < (1 << bw)) h = __floats2half2_rn(__ldg(cent + index), __ldg(cent + index));
  return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_half(uint32_t a) {
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(h) : "r"(a));
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same instruction as a pure function of its operands: the compiler may
// move it between the (ordered) shared-memory loads around it.
__device__ __forceinline__ void mma16816_free(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}

// ---- table lookups ----------------------------------------------------------
// `sel` carries 0x10000, the side bit (values: 0x80) and the lane's bank.
// 4-bit: entry of byte K (0..3) of `word`, a half2 of the byte's two codes.
template <int K> __device__ __forceinline__ uint32_t lut_addr(uint32_t word, uint32_t sel) {
  return __byte_perm(word, sel, 0x7604 | (K << 4));
}
template <int K> __device__ __forceinline__ uint32_t lut_byte(uint32_t word, uint32_t sel) {
  return lds32(lut_addr<K>(word, sel));
}
// 6/8-bit: entry {c, c} of code I of the bit stream held in w[0..NW).
template <int BW, int I, int NW>
__device__ __forceinline__ uint32_t lut_code(const uint32_t (&w)[NW], uint32_t sel) {
  constexpr int bit = I * BW, word = bit / 32, off = bit % 32;
  static_assert(word < NW, "code outside the words held");
  if constexpr (BW == 8) {
    return lds32(__byte_perm(w[word], sel, 0x7604 | ((off / 8) << 4)));
  } else {
    constexpr uint32_t mask = ((1u << BW) - 1u) << 8;
    uint32_t x;
    if constexpr (off + BW <= 32) {
      x = off >= 8 ? (w[word] >> (off >= 8 ? off - 8 : 0)) : (w[word] << (off < 8 ? 8 - off : 0));
    } else {                                     // the code straddles two words
      x = __funnelshift_r(w[word], w[word + 1 < NW ? word + 1 : word], off - 8);
    }
    return lds32((x & mask) | sel);
  }
}
// low half of x joined with the high half of y
__device__ __forceinline__ uint32_t join(uint32_t x, uint32_t y) {
  return __byte_perm(x, y, 0x7610);
}

// Words of a lane's share of a packed row: NBYTES at shared address a.
template <int NBYTES>
__device__ __forceinline__ void load_words(uint32_t a, uint32_t (&w)[NBYTES / 4]) {
  if constexpr (NBYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < NBYTES / 16; ++i) {
      const uint4 v = lds128(a + 16 * i);
      w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
  } else if constexpr (NBYTES % 8 == 0) {
#pragma unroll
    for (int i = 0; i < NBYTES / 8; ++i) {
      const uint2 v = lds64(a + 8 * i);
      w[2 * i] = v.x; w[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NBYTES / 4; ++i) w[i] = lds32(a + 4 * i);
  }
}

}  // namespace mma

using namespace mma;

// A-fragment registers of the score MMA for contraction step KS (0..7): the
// lane holds 32 codes (coordinates 32t..32t+31) of token rows g (w0) and g+8
// (w1); step KS consumes codes 4KS..4KS+3 of each.
template <int BW, int KS, int NW>
__device__ __forceinline__ void key_fragment(const uint32_t (&w0)[NW], const uint32_t (&w1)[NW],
                                             uint32_t sel, uint32_t (&a)[4]) {
  if constexpr (BW == 4) {
    constexpr int j = KS / 2, e = 2 * (KS % 2);
    a[0] = lut_byte<e>(w0[j], sel);
    a[1] = lut_byte<e>(w1[j], sel);
    a[2] = lut_byte<e + 1>(w0[j], sel);
    a[3] = lut_byte<e + 1>(w1[j], sel);
  } else {
    constexpr int i = 4 * KS;
    a[0] = join(lut_code<BW, i>(w0, sel), lut_code<BW, i + 1>(w0, sel));
    a[1] = join(lut_code<BW, i>(w1, sel), lut_code<BW, i + 1>(w1, sel));
    a[2] = join(lut_code<BW, i + 2>(w0, sel), lut_code<BW, i + 3>(w0, sel));
    a[3] = join(lut_code<BW, i + 2>(w1, sel), lut_code<BW, i + 3>(w1, sel));
  }
}

}  // namespace wtq
