/* Second, independent CPU statement of the rotate+quantise row kernel, in plain C.
 *
 * Test infrastructure: it is compiled by the build step and loaded only by tests, to cross-check the NumPy
 * restatement (oracle/rotq8_ref.py). It keeps the reference kernel's data distribution explicit instead of
 * vectorising it away: a rotation block is spread over `block / 8` lanes holding eight consecutive channels
 * each (kernels/ops.metal:9-10 of the reference); three butterfly stages run inside a lane (ops.metal:19-31),
 * the remaining log2(block/8) stages pair lane l with lane l ^ s, the lower lane keeping v + o and the upper
 * lane o - v (ops.metal:34-44); one multiply by the normaliser follows (ops.metal:46; 1/sqrt(block) in fp32).
 * Then amax over the row, scale = amax / 127 (1 if the row is all zero), rs = 1 / scale and
 * code = rint(v * rs) (ops.metal:315-327).
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared oracle/rotq8_witness.c -o oracle/_build/librotq8_witness.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define LANE_VALUES 8

static void lane_butterflies(float *v) {
  for (int s = 1; s < LANE_VALUES; s <<= 1)
    for (int i = 0; i < LANE_VALUES; i++)
      if ((i & s) == 0) {
        const float a = v[i], b = v[i + s];
        v[i] = a + b;
        v[i + s] = a - b;
      }
}

/* lanes[l][i]: value i of lane l; n_lanes = block / 8 */
static void block_transform(float (*lanes)[LANE_VALUES], int n_lanes, float normaliser) {
  float other[32][LANE_VALUES];
  for (int l = 0; l < n_lanes; l++) lane_butterflies(lanes[l]);
  for (int s = 1; s < n_lanes; s <<= 1) {
    for (int l = 0; l < n_lanes; l++)
      for (int i = 0; i < LANE_VALUES; i++) other[l][i] = lanes[l ^ s][i]; /* the shuffle: every lane reads first */
    for (int l = 0; l < n_lanes; l++)
      for (int i = 0; i < LANE_VALUES; i++)
        lanes[l][i] = (l & s) ? other[l][i] - lanes[l][i] : lanes[l][i] + other[l][i];
  }
  for (int l = 0; l < n_lanes; l++)
    for (int i = 0; i < LANE_VALUES; i++) lanes[l][i] *= normaliser;
}

static float silu(float x) { return x / (1.0f + expf(-x)); }

/* x: fp32 rows (already widened from bf16/fp16), row stride x_stride elements; mode 1: gates at column D + c.
 * rotated (may be NULL) receives the fp32 rotated rows [M][D]. Returns 0, or -1 on bad sizes. */
int rotq8_witness(const float *x, int M, int D, long x_stride, int block, int mode, int8_t *codes, float *scales,
                  float *rotated) {
  if (block < 8 || block > 256 || (block & (block - 1)) || D % block) return -1;
  const int n_lanes = block / LANE_VALUES;
  const float normaliser = (float)(1.0 / sqrt((double)block));
  float *row = (float *)malloc(sizeof(float) * (size_t)D);
  if (!row) return -1;
  for (int m = 0; m < M; m++) {
    const float *src = x + (size_t)m * x_stride;
    float amax = 0.0f;
    for (int b0 = 0; b0 < D; b0 += block) {
      float lanes[32][LANE_VALUES];
      for (int l = 0; l < n_lanes; l++)
        for (int i = 0; i < LANE_VALUES; i++) {
          const int c = b0 + l * LANE_VALUES + i;
          float val = src[c];
          if (mode == 1) val *= silu(src[D + c]);
          lanes[l][i] = val;
        }
      block_transform(lanes, n_lanes, normaliser);
      for (int l = 0; l < n_lanes; l++)
        for (int i = 0; i < LANE_VALUES; i++) {
          const float v = lanes[l][i];
          row[b0 + l * LANE_VALUES + i] = v;
          amax = fmaxf(amax, fabsf(v));
        }
    }
    const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
    const float rs = 1.0f / scale;
    for (int c = 0; c < D; c++) {
      if (rotated) rotated[(size_t)m * D + c] = row[c];
      codes[(size_t)m * D + c] = (int8_t)rintf(row[c] * rs);
    }
    scales[m] = scale;
  }
  free(row);
  return 0;
}
