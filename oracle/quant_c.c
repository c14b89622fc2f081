/*
 * Oracle (test infrastructure): the static per-head INT8 quantiser restated in plain C, as an independent
 * check of the PyTorch restatement in oracle/quant.py.  Follows src/quant.py:37-40 of the reference:
 * q = clamp(round_half_even(x / scale), -127, 127) with the quotient formed in IEEE binary32, and
 * src/triton_ops/int8_cache_write.py:152-183 for the slot scatter (slot < 0 skips the token).
 *
 * Build: gcc -O2 -shared -fPIC -fno-fast-math -o oracle/_build/libquant_c.so oracle/quant_c.c -lm
 */
#include <math.h>
#include <stdint.h>

static int8_t quant_one(float x, float scale) {
  volatile float q = x / scale;        /* binary32 quotient, no excess precision */
  float r = nearbyintf(q);             /* default rounding mode: to nearest, ties to even */
  if (r > 127.0f) r = 127.0f;
  if (r < -127.0f) r = -127.0f;
  if (r != r) return 0;                /* NaN: what a float -> int8 cast gives on x86 */
  return (int8_t)r;
}

/* x [tokens, heads, dim] float32 -> q [tokens, heads, dim] int8, one scale per head */
void oracle_static_quant(const float* x, const float* scale, int8_t* q, int64_t tokens, int heads, int dim,
                         int floor_scale) {
  for (int64_t t = 0; t < tokens; ++t)
    for (int h = 0; h < heads; ++h) {
      float s = scale[h];
      if (floor_scale && s < 1e-6f) s = 1e-6f;
      for (int d = 0; d < dim; ++d) {
        const int64_t i = (t * heads + h) * dim + d;
        q[i] = quant_one(x[i], s);
      }
    }
}

/* scatter write into cache [num_blocks, block_size, heads, dim]; later tokens win on a repeated slot */
void oracle_cache_write(const float* x, const float* scale, int8_t* cache, const int64_t* slots, int64_t tokens,
                        int heads, int dim, int64_t num_blocks, int block_size, int floor_scale) {
  const int64_t row = (int64_t)heads * dim;
  for (int64_t t = 0; t < tokens; ++t) {
    const int64_t slot = slots[t];
    if (slot < 0 || slot >= num_blocks * block_size) continue;
    for (int h = 0; h < heads; ++h) {
      float s = scale[h];
      if (floor_scale && s < 1e-6f) s = 1e-6f;
      for (int d = 0; d < dim; ++d) cache[slot * row + h * dim + d] = quant_one(x[t * row + h * dim + d], s);
    }
  }
}
