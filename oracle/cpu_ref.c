/* Pinned-order C restatement of the k2b page quantizer (test infrastructure only).
 *
 * The numpy oracle (bmx_oracle.py) follows the reference and therefore leaves the order of its
 * float32 reductions to BLAS; the CUDA append kernels fix that order.  This file repeats the CUDA
 * order step for step in plain C (fmaf = one rounding, as on the GPU), so that the bytes a GPU append
 * writes can be compared for equality, not just statistically:
 *   projection  Us[r,i] = sum over channels c ascending (heads ascending) of fmaf(M[r,c], V[c,i], acc)
 *   low rank    L[r,c]  = sum over i ascending of fmaf(half(Us[r,i]), half(V[c,i]), acc)
 *   residual    R = M - L ; per channel and group of `group` tokens scale = max(absmax, 1e-12) / qmax,
 *               code = clamp(rint(R / scale), -qmax-1, qmax)            (bmx src/bmx/quant/rtn.py:34-44)
 *   values      per (token, head): ss = 4-element fmaf chains per lane, then a 5-level xor tree over the
 *               32 lanes; n = half(max(sqrt(ss), 1e-12)); u = v / n * sign; FWHT butterflies h = 1..64
 *               (low = a + b, high = a - b), / float(sqrt(128)); idx = #{mid < y * float(sqrt(128))}
 *               (bmx src/bmx/cache/codecs.py:616-636, src/bmx/quant/hadamard.py:12-33)
 * Build: make -C oracle   ->  oracle/libcpu_ref.so
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define D 128

static uint16_t f2h(float f) { /* float32 -> fp16 bits, round to nearest even */
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u, mant = x & 0x7FFFFFu;
  int32_t exp = (int32_t)((x >> 23) & 0xFF);
  if (exp == 0xFF) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0));
  int32_t e = exp - 127 + 15;
  if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    mant |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - e), half = 1u << (shift - 1), rem = mant & ((1u << shift) - 1u);
    uint32_t m = mant >> shift;
    if (rem > half || (rem == half && (m & 1u))) m++;
    return (uint16_t)(sign | m);
  }
  uint32_t m = mant >> 13, rem = mant & 0x1FFFu;
  uint32_t out = sign | ((uint32_t)e << 10) | m;
  if (rem > 0x1000u || (rem == 0x1000u && (m & 1u))) out++;
  return (uint16_t)out;
}
static float h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, mant = h & 0x3FFu, x;
  if (exp == 0) {
    if (mant == 0) x = sign;
    else {
      int e = -1;
      do { mant <<= 1; e++; } while (!(mant & 0x400u));
      x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3FFu) << 13);
    }
  } else if (exp == 0x1F) x = sign | 0x7F800000u | (mant << 13);
  else x = sign | ((exp - 15 + 127) << 23) | (mant << 13);
  float f;
  memcpy(&f, &x, 4);
  return f;
}
static float hround(float f) { return h2f(f2h(f)); }

/* One page of one sequence, all heads.  M, Vv: (page, C) float32 with C = h_kv*128 (bmx to_matrix layout).
 * basis: (C, rank) float32.  Outputs in the layout of bmx's build_kv_stacked_k2b:
 *   us (n_coef_heads, page, rank) fp16 bits; res (C, page) int8; res_scale (C, page/group) fp16 bits;
 *   v_idx (page, C) uint8; v_norm (page, h_kv) fp16 bits. */
void k2b_quant_page_ref(const float* M, const float* Vv, const float* basis, const float* signs, const float* codebook,
                        int h_kv, int page, int rank, int group, int n_coef_heads, int kbits, uint16_t* us, int8_t* res,
                        uint16_t* res_scale, uint8_t* v_idx, uint16_t* v_norm) {
  const int C = h_kv * D, ngrp = page / group;
  const float qmax = (float)((1 << (kbits - 1)) - 1);
  for (int ch = 0; ch < n_coef_heads; ++ch) {
    const int h0 = n_coef_heads == 1 ? 0 : ch, nh = n_coef_heads == 1 ? h_kv : 1;
    for (int r = 0; r < page; ++r)
      for (int i = 0; i < rank; ++i) {
        float acc = 0.f;
        for (int h = h0; h < h0 + nh; ++h)
          for (int c = 0; c < D; ++c) acc = fmaf(M[(size_t)r * C + h * D + c], basis[(size_t)(h * D + c) * rank + i], acc);
        us[((size_t)ch * page + r) * rank + i] = f2h(acc);
      }
  }
  for (int h = 0; h < h_kv; ++h) {
    const int ch = n_coef_heads == 1 ? 0 : h;
    for (int c = 0; c < D; ++c) {
      const int cg = h * D + c;
      for (int g = 0; g < ngrp; ++g) {
        float amax = 0.f;
        for (int pass = 0; pass < 2; ++pass) {
          const float scale = fmaxf(amax, 1e-12f) / qmax;
          if (pass == 1) res_scale[(size_t)cg * ngrp + g] = f2h(scale);
          for (int r = g * group; r < (g + 1) * group; ++r) {
            float L = 0.f;
            for (int i = 0; i < rank; ++i)
              L = fmaf(h2f(us[((size_t)ch * page + r) * rank + i]), hround(basis[(size_t)cg * rank + i]), L);
            const float R = M[(size_t)r * C + cg] - L;
            if (pass == 0) amax = fmaxf(amax, fabsf(R));
            else {
              float q = rintf(R / scale);
              q = fminf(fmaxf(q, -qmax - 1.f), qmax);
              res[(size_t)cg * page + r] = (int8_t)q;
            }
          }
        }
      }
    }
    const float m0 = (codebook[0] + codebook[1]) / 2.f, m1 = (codebook[1] + codebook[2]) / 2.f, m2 = (codebook[2] + codebook[3]) / 2.f;
    const float sqrt_d = 11.313708498984761f;
    for (int r = 0; r < page; ++r) {
      float x[D], lane[32];
      for (int c = 0; c < D; ++c) x[c] = Vv[(size_t)r * C + h * D + c];
      for (int l = 0; l < 32; ++l) {
        float ss = 0.f;
        for (int k = 0; k < 4; ++k) ss = fmaf(x[4 * l + k], x[4 * l + k], ss);
        lane[l] = ss;
      }
      for (int m = 16; m >= 1; m >>= 1) {
        float t[32];
        for (int l = 0; l < 32; ++l) t[l] = lane[l] + lane[l ^ m];
        memcpy(lane, t, sizeof(t));
      }
      const float n = hround(fmaxf(sqrtf(lane[0]), 1e-12f));
      v_norm[(size_t)r * h_kv + h] = f2h(n);
      for (int c = 0; c < D; ++c) x[c] = (x[c] / n) * signs[c];
      for (int hh = 1; hh < D; hh <<= 1)
        for (int i = 0; i < D; i += 2 * hh)
          for (int k = i; k < i + hh; ++k) {
            const float a = x[k], b = x[k + hh];
            x[k] = a + b;
            x[k + hh] = a - b;
          }
      for (int c = 0; c < D; ++c) {
        const float y = (x[c] / sqrt_d) * sqrt_d;
        v_idx[(size_t)r * C + h * D + c] = (uint8_t)((y > m0) + (y > m1) + (y > m2));
      }
    }
  }
}
