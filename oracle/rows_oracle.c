/* CPU restatement of the bandwidth-bound configuration, for timing and for
 * parity checks at sizes where the numpy oracle is slow.  TEST INFRASTRUCTURE
 * ONLY: nothing in the product links or calls this file.
 *
 * One pass per output with no fusion across outputs, which is how the
 * reference's evaluator walks the graph node by node
 * (nx/lib/nx/defn/evaluator.ex:363-388): reduce_max (nx/lib/nx/binary_backend.ex:1344-1355),
 * exp(x - max), sum (:1316-1324), Nx.logsumexp (nx/lib/nx.ex:18400-18433), the
 * softmax division, argmax with the lowest index on ties (:1415-1431) and the
 * chain tanh(x*0.5+0.1)*sigmoid(x).  Elementwise arithmetic is f32 (XLA-style
 * numerics; the f64 BinaryBackend mode lives in nx_oracle.py); the two row sums
 * are accumulated in double and rounded once, as the reference's reducer does
 * (bin_reduce folds Erlang floats, nx/lib/nx/binary_backend.ex:2342-2360): a
 * sequential f32 sum over 32768 terms would carry an error of the order of the
 * tolerance itself and could not serve as the expected value.  Rows are
 * independent and are spread over OpenMP threads.
 */
#include <math.h>
#include <stdint.h>
#include <omp.h>

int rows_oracle_threads(void) { return omp_get_max_threads(); }
void rows_oracle_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

void rows_oracle(const float *x, int64_t rows, int64_t cols, float *rowmax, float *e, float *sum,
                 float *lse, float *softmax, int32_t *argmax, float *chain) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *er = e + r * cols, *sr = softmax + r * cols, *cr = chain + r * cols;
    /* reduce_max: NaN propagates */
    float m = -INFINITY;
    int has_nan = 0;
    for (int64_t c = 0; c < cols; ++c) {
      if (xr[c] != xr[c]) has_nan = 1;
      if (xr[c] > m) m = xr[c];
    }
    if (has_nan) m = NAN;
    rowmax[r] = m;
    /* exp(x - max) materialised, then its sum */
    for (int64_t c = 0; c < cols; ++c) er[c] = expf(xr[c] - m);
    double sd = 0.0;
    for (int64_t c = 0; c < cols; ++c) sd += (double)er[c];
    const float s = (float)sd;
    sum[r] = s;
    /* logsumexp: the max is replaced by 0 when it is infinite */
    float m2 = isinf(m) ? 0.f : m;
    double s2d = 0.0;
    for (int64_t c = 0; c < cols; ++c) s2d += (double)expf(xr[c] - m2);
    lse[r] = logf((float)s2d) + m2;
    for (int64_t c = 0; c < cols; ++c) sr[c] = er[c] / s;
    /* argmax: a candidate replaces the current one if strictly greater or NaN */
    int64_t best = 0;
    float bv = xr[0];
    for (int64_t c = 1; c < cols; ++c) {
      float v = xr[c];
      if (v != v || (!(bv != bv) && v > bv)) { bv = v; best = c; }
    }
    argmax[r] = (int32_t)best;
    for (int64_t c = 0; c < cols; ++c) cr[c] = tanhf(xr[c] * 0.5f + 0.1f) * (1.0f / (1.0f + expf(-xr[c])));
  }
}
