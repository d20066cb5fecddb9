/*
 * CPU restatement of portDNN's operator semantics.  TEST INFRASTRUCTURE ONLY:
 * this file is the checker the CUDA kernels are compared against (and the CPU
 * arm of the benchmark).  Nothing in the shipped library calls it.
 *
 * Parity status: PINNED.  oracle/pin_oracle.py replays the reference's own
 * known-answer vectors (its generated gtest sources for conv2d,
 * depthwise_conv2d and pooling, plus the hand-written pointwise / bias /
 * matmul cases) through these functions; the committed subset lives in
 * tests/golden/.
 *
 * Each routine states the reference source it follows (paths are relative to
 * the portDNN project root).  The loops here are written from the
 * mathematical definition, not transcribed: the reference assigns one SYCL
 * work-item per output element, whereas these are plain nested loops with
 * OpenMP over the outermost independent index.
 *
 * Layouts (row-major, last index fastest): activations NHWC, conv filter HWCF
 * [R][S][C/groups][K], depthwise filter [R][S][C][mult], matrices row-major.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

/* Mirror of sycldnn::conv2d::Conv2DParams (include/portdnn/conv2d/params.h:32-112):
 * same field order, all int; the three trailing enums are carried as ints. */
typedef struct {
  int channels, features, batch, in_rows, in_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int out_rows, out_cols, pad_rows, pad_cols;
  int dilation_rows, dilation_cols, groups;
  int input_format, filter_format, group_format;
} OrcConvParams;

/* Mirror of sycldnn::depthwise_conv2d::DepthwiseConv2DParams
 * (include/portdnn/depthwise_conv2d/params.h:33-94). */
typedef struct {
  int channels, channel_multiplier, batch, in_rows, in_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int out_rows, out_cols, pad_rows, pad_cols;
} OrcDepthwiseParams;

/* Mirror of sycldnn::pooling::PoolingParams (include/portdnn/pooling/params.h:30-73). */
typedef struct {
  int in_rows, in_cols, out_rows, out_cols;
  int window_rows, window_cols, stride_rows, stride_cols;
  int batch, channels, pad_rows, pad_cols;
  int input_format;
} OrcPoolParams;

enum { ORC_FORWARD = 0, ORC_INPUT_BACKPROP = 1, ORC_FILTER_BACKPROP = 2 };
enum { ORC_POOL_MAX = 0, ORC_POOL_MAX_WITH_NAN = 1, ORC_POOL_AVERAGE = 2 };
enum { ORC_ADD = 0, ORC_SUB = 1, ORC_MUL = 2, ORC_DIV = 3 };
enum { ORC_RELU = 0, ORC_TANH = 1, ORC_EXP = 3, ORC_LOG = 4, ORC_FLOOR = 5, ORC_SQRT = 6 };  /* 2 is the GPU side's ReLU6 */

/* ------------------------------------------------------------------------- */
/* conv2d                                                                    */
/* ------------------------------------------------------------------------- */

/* Forward: y[n,oh,ow,k] = sum_{r,s,c} x[n, oh*st-pad+r, ow*st-pad+s, c] * w[r,s,c,k],
 * out-of-range x reads as zero.  Follows src/conv2d/direct/kernels_nhwc.h:62-130
 * (cross-correlation, implicit high-side padding).  Groups follow the im2col
 * driver's convention (include/portdnn/internal/conv2d/im2col.h:90-137): group g
 * reads channels [g*C/G,(g+1)*C/G) and writes features [g*K/G,(g+1)*K/G); the
 * filter is [R][S][C/G][K].  With group_format INTERLEAVED the group is the fastest
 * index of the channel and feature axes instead (channel c of group g is element
 * c*G+g of a pixel, feature k of group g is element k*G+g of the filter's last axis
 * and of an output pixel), as test/conv2d/group_convolution_fixture.h:41-77 lays the
 * tensors out and include/portdnn/batch_format.h:33-47 defines it.  Accumulates in double. */
static void conv_forward(const float* x, const float* w, float* y, const OrcConvParams* p) {
  const int C = p->channels, K = p->features, G = p->groups > 0 ? p->groups : 1;
  const int Cg = C / G, Kg = K / G;
  /* element strides of (group, index within the group) on the channel and feature axes */
  const int il = p->group_format == 1;
  const int cgs = il ? 1 : Cg, ccs = il ? G : 1, kgs = il ? 1 : Kg, kks = il ? G : 1;
  const long rows_total = (long)p->batch * p->out_rows;
#pragma omp parallel
  {
    double* acc = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(static)
    for (long nr = 0; nr < rows_total; ++nr) {
      const int n = (int)(nr / p->out_rows), oh = (int)(nr % p->out_rows);
      for (int ow = 0; ow < p->out_cols; ++ow) {
        for (int k = 0; k < K; ++k) acc[k] = 0.0;
        for (int r = 0; r < p->window_rows; ++r) {
          const int ih = oh * p->stride_rows - p->pad_rows + r;
          if (ih < 0 || ih >= p->in_rows) continue;
          for (int s = 0; s < p->window_cols; ++s) {
            const int iw = ow * p->stride_cols - p->pad_cols + s;
            if (iw < 0 || iw >= p->in_cols) continue;
            const float* xp = x + (((size_t)n * p->in_rows + ih) * p->in_cols + iw) * C;
            const float* wp = w + ((size_t)r * p->window_cols + s) * Cg * K;
            for (int g = 0; g < G; ++g) {
              for (int c = 0; c < Cg; ++c) {
                const double xv = xp[g * cgs + c * ccs];
                const float* wk = wp + (size_t)c * K + g * kgs;
                double* ak = acc + g * kgs;
                for (int k = 0; k < Kg; ++k) ak[k * kks] += xv * (double)wk[k * kks];
              }
            }
          }
        }
        float* yp = y + (((size_t)n * p->out_rows + oh) * p->out_cols + ow) * K;
        for (int k = 0; k < K; ++k) yp[k] = (float)acc[k];
      }
    }
    free(acc);
  }
}

/* Input backprop: dx[n,h,w,c] = sum_k sum_{(oh,r): oh*st-pad+r=h} sum_{(ow,s): ow*st-pad+s=w}
 * dy[n,oh,ow,k] * w[r,s,c,k].  Follows src/conv2d/direct/kernels_nhwc.h:206-278 with the
 * parameter remap of src/conv2d/direct/kernel_params.h:36-40 (the reference walks a
 * mirrored filter with pad' = window-1-pad; this is the same sum written from the
 * forward relation). */
static void conv_input_backprop(const float* dy, const float* w, float* dx, const OrcConvParams* p) {
  const int C = p->channels, K = p->features;
  const long rows_total = (long)p->batch * p->in_rows;
#pragma omp parallel
  {
    double* acc = (double*)malloc(sizeof(double) * (size_t)C);
#pragma omp for schedule(static)
    for (long nr = 0; nr < rows_total; ++nr) {
      const int n = (int)(nr / p->in_rows), h = (int)(nr % p->in_rows);
      for (int wi = 0; wi < p->in_cols; ++wi) {
        for (int c = 0; c < C; ++c) acc[c] = 0.0;
        for (int r = 0; r < p->window_rows; ++r) {
          const int th = h + p->pad_rows - r;
          if (th < 0 || th % p->stride_rows) continue;
          const int oh = th / p->stride_rows;
          if (oh >= p->out_rows) continue;
          for (int s = 0; s < p->window_cols; ++s) {
            const int tw = wi + p->pad_cols - s;
            if (tw < 0 || tw % p->stride_cols) continue;
            const int ow = tw / p->stride_cols;
            if (ow >= p->out_cols) continue;
            const float* dyp = dy + (((size_t)n * p->out_rows + oh) * p->out_cols + ow) * K;
            const float* wp = w + ((size_t)r * p->window_cols + s) * C * K;
            for (int c = 0; c < C; ++c) {
              const float* wk = wp + (size_t)c * K;
              double sum = 0.0;
              for (int k = 0; k < K; ++k) sum += (double)dyp[k] * (double)wk[k];
              acc[c] += sum;
            }
          }
        }
        float* dxp = dx + (((size_t)n * p->in_rows + h) * p->in_cols + wi) * C;
        for (int c = 0; c < C; ++c) dxp[c] = (float)acc[c];
      }
    }
    free(acc);
  }
}

/* Filter backprop: dW[r,s,c,k] = sum_{n,oh,ow} x[n, oh*st-pad+r, ow*st-pad+s, c] * dy[n,oh,ow,k].
 * Follows src/conv2d/direct/kernels_nhwc.h:356-420 (the reference swaps the roles of
 * output size and window, src/conv2d/direct/kernel_params.h:42-52; same sum). */
static void conv_filter_backprop(const float* x, const float* dy, float* dw, const OrcConvParams* p) {
  const int C = p->channels, K = p->features;
  const int taps = p->window_rows * p->window_cols;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int t = 0; t < taps; ++t) {
    for (int c = 0; c < C; ++c) {
      const int r = t / p->window_cols, s = t % p->window_cols;
      double* acc = (double*)calloc((size_t)K, sizeof(double));
      for (int n = 0; n < p->batch; ++n) {
        for (int oh = 0; oh < p->out_rows; ++oh) {
          const int ih = oh * p->stride_rows - p->pad_rows + r;
          if (ih < 0 || ih >= p->in_rows) continue;
          for (int ow = 0; ow < p->out_cols; ++ow) {
            const int iw = ow * p->stride_cols - p->pad_cols + s;
            if (iw < 0 || iw >= p->in_cols) continue;
            const double xv = x[(((size_t)n * p->in_rows + ih) * p->in_cols + iw) * C + c];
            const float* dyp = dy + (((size_t)n * p->out_rows + oh) * p->out_cols + ow) * K;
            for (int k = 0; k < K; ++k) acc[k] += xv * (double)dyp[k];
          }
        }
      }
      float* out = dw + ((size_t)t * C + c) * K;
      for (int k = 0; k < K; ++k) out[k] = (float)acc[k];
      free(acc);
    }
  }
}

/* Entry: argument slots follow conv2d::launch (include/portdnn/conv2d/launch.h:59-72):
 * Forward (x, w, y); InputBackprop (dy, w, dx); FilterBackprop (x, dy, dW).
 * Returns 0, or -1 for a parameter set the reference's validate_params
 * (include/portdnn/internal/conv2d/launch.h:42-97) rejects or this oracle does
 * not cover (NCHW, FHWC). */
int orc_conv2d(int pass, const float* in, const float* fil, float* out, const OrcConvParams* p) {
  if (p->dilation_rows != 1 || p->dilation_cols != 1) return -1;
  if (p->input_format != 0 || p->filter_format != 0) return -1;
  const int G = p->groups > 0 ? p->groups : 1;
  if (G != 1 && pass != ORC_FORWARD) return -1;
  if (p->channels % G || p->features % G) return -1;
  if (p->group_format != 0 && (p->group_format != 1 || G == 1)) return -1;
  switch (pass) {
    case ORC_FORWARD: conv_forward(in, fil, out, p); return 0;
    case ORC_INPUT_BACKPROP: conv_input_backprop(in, fil, out, p); return 0;
    case ORC_FILTER_BACKPROP: conv_filter_backprop(in, fil, out, p); return 0;
  }
  return -1;
}

/* Forward convolution with float accumulation, used only as the timed CPU
 * baseline: same definition as conv_forward (src/conv2d/direct/kernels_nhwc.h:62-130,
 * which also accumulates in the data type), inner loop over contiguous features so
 * that the compiler vectorises it. groups == 1 only. */
int orc_conv2d_forward_f32(const float* x, const float* w, float* y, const OrcConvParams* p) {
  const int C = p->channels, K = p->features;
  const long pix_total = (long)p->batch * p->out_rows * p->out_cols;
#pragma omp parallel for schedule(static)
  for (long pix = 0; pix < pix_total; ++pix) {
    const int ow = (int)(pix % p->out_cols);
    const int oh = (int)((pix / p->out_cols) % p->out_rows);
    const int n = (int)(pix / ((long)p->out_cols * p->out_rows));
    float* yp = y + (size_t)pix * K;
    for (int k = 0; k < K; ++k) yp[k] = 0.f;
    for (int r = 0; r < p->window_rows; ++r) {
      const int ih = oh * p->stride_rows - p->pad_rows + r;
      if (ih < 0 || ih >= p->in_rows) continue;
      for (int s = 0; s < p->window_cols; ++s) {
        const int iw = ow * p->stride_cols - p->pad_cols + s;
        if (iw < 0 || iw >= p->in_cols) continue;
        const float* xp = x + (((size_t)n * p->in_rows + ih) * p->in_cols + iw) * C;
        const float* wp = w + ((size_t)r * p->window_cols + s) * C * K;
        for (int c = 0; c < C; ++c) {
          const float xv = xp[c];
          const float* wk = wp + (size_t)c * K;
          for (int k = 0; k < K; ++k) yp[k] += xv * wk[k];
        }
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* depthwise conv2d                                                          */
/* ------------------------------------------------------------------------- */

/* Follows src/depthwise_conv2d/kernels.h:58-125 (forward), :154-225 (input
 * backprop), :259-360 (filter backprop) and src/depthwise_conv2d/kernel_params.h:29-49.
 * Output channel of (c, m) is c*mult+m; the filter is [R][S][C][mult]. */
int orc_depthwise_conv2d(int pass, const float* in, const float* fil, float* out,
                         const OrcDepthwiseParams* p) {
  const int C = p->channels, M = p->channel_multiplier, F = C * M;
  if (pass == ORC_FORWARD) {
    const long total = (long)p->batch * p->out_rows * p->out_cols;
#pragma omp parallel for schedule(static)
    for (long pix = 0; pix < total; ++pix) {
      const int ow = (int)(pix % p->out_cols);
      const int oh = (int)((pix / p->out_cols) % p->out_rows);
      const int n = (int)(pix / ((long)p->out_cols * p->out_rows));
      for (int f = 0; f < F; ++f) {
        const int c = f / M;
        double acc = 0.0;
        for (int r = 0; r < p->window_rows; ++r) {
          const int ih = oh * p->stride_rows - p->pad_rows + r;
          if (ih < 0 || ih >= p->in_rows) continue;
          for (int s = 0; s < p->window_cols; ++s) {
            const int iw = ow * p->stride_cols - p->pad_cols + s;
            if (iw < 0 || iw >= p->in_cols) continue;
            acc += (double)in[(((size_t)n * p->in_rows + ih) * p->in_cols + iw) * C + c] *
                   (double)fil[((size_t)r * p->window_cols + s) * F + f];
          }
        }
        out[(size_t)pix * F + f] = (float)acc;
      }
    }
    return 0;
  }
  if (pass == ORC_INPUT_BACKPROP) {
    const long total = (long)p->batch * p->in_rows * p->in_cols;
#pragma omp parallel for schedule(static)
    for (long pix = 0; pix < total; ++pix) {
      const int wi = (int)(pix % p->in_cols);
      const int h = (int)((pix / p->in_cols) % p->in_rows);
      const int n = (int)(pix / ((long)p->in_cols * p->in_rows));
      for (int c = 0; c < C; ++c) {
        double acc = 0.0;
        for (int r = 0; r < p->window_rows; ++r) {
          const int th = h + p->pad_rows - r;
          if (th < 0 || th % p->stride_rows) continue;
          const int oh = th / p->stride_rows;
          if (oh >= p->out_rows) continue;
          for (int s = 0; s < p->window_cols; ++s) {
            const int tw = wi + p->pad_cols - s;
            if (tw < 0 || tw % p->stride_cols) continue;
            const int ow = tw / p->stride_cols;
            if (ow >= p->out_cols) continue;
            const float* dyp = in + (((size_t)n * p->out_rows + oh) * p->out_cols + ow) * F + (size_t)c * M;
            const float* wp = fil + ((size_t)r * p->window_cols + s) * F + (size_t)c * M;
            for (int m = 0; m < M; ++m) acc += (double)dyp[m] * (double)wp[m];
          }
        }
        out[(size_t)pix * C + c] = (float)acc;
      }
    }
    return 0;
  }
  if (pass == ORC_FILTER_BACKPROP) {
    const int taps = p->window_rows * p->window_cols;
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int t = 0; t < taps; ++t) {
      for (int f = 0; f < F; ++f) {
        const int r = t / p->window_cols, s = t % p->window_cols, c = f / M;
        double acc = 0.0;
        for (int n = 0; n < p->batch; ++n)
          for (int oh = 0; oh < p->out_rows; ++oh) {
            const int ih = oh * p->stride_rows - p->pad_rows + r;
            if (ih < 0 || ih >= p->in_rows) continue;
            for (int ow = 0; ow < p->out_cols; ++ow) {
              const int iw = ow * p->stride_cols - p->pad_cols + s;
              if (iw < 0 || iw >= p->in_cols) continue;
              acc += (double)in[(((size_t)n * p->in_rows + ih) * p->in_cols + iw) * C + c] *
                     (double)fil[(((size_t)n * p->out_rows + oh) * p->out_cols + ow) * F + f];
            }
          }
        out[(size_t)t * F + f] = (float)acc;
      }
    }
    return 0;
  }
  return -1;
}

/* ------------------------------------------------------------------------- */
/* pooling                                                                   */
/* ------------------------------------------------------------------------- */

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

/* Forward pooling, NHWC.  The window is clamped to the image, so Average divides
 * by the number of valid elements (src/pooling/kernels.h:61-101).  Max starts from
 * lowest() and keeps val only if val > max (NaN never wins); MaxWithNan also takes
 * a NaN and then keeps it (src/pooling/operators_impl.h:27-87).  Average sums in
 * float in row-major window order, like the reference's accumulator. */
int orc_pool_forward(int op, const float* x, float* y, const OrcPoolParams* p) {
  const int C = p->channels;
  const long total = (long)p->batch * p->out_rows * p->out_cols;
#pragma omp parallel for schedule(static)
  for (long pix = 0; pix < total; ++pix) {
    const int ow = (int)(pix % p->out_cols);
    const int oh = (int)((pix / p->out_cols) % p->out_rows);
    const int n = (int)(pix / ((long)p->out_cols * p->out_rows));
    int r0 = oh * p->stride_rows - p->pad_rows, c0 = ow * p->stride_cols - p->pad_cols;
    const int r1 = imin(r0 + p->window_rows, p->in_rows), c1 = imin(c0 + p->window_cols, p->in_cols);
    r0 = imax(r0, 0);
    c0 = imax(c0, 0);
    for (int c = 0; c < C; ++c) {
      float best = -FLT_MAX, sum = 0.f;
      int tally = 0;
      for (int r = r0; r < r1; ++r)
        for (int cc = c0; cc < c1; ++cc) {
          const float v = x[(((size_t)n * p->in_rows + r) * p->in_cols + cc) * C + c];
          if (op == ORC_POOL_MAX) {
            if (v > best) best = v;
          } else if (op == ORC_POOL_MAX_WITH_NAN) {
            if (isnan(v) || v > best) best = v;
          } else {
            sum += v;
            ++tally;
          }
        }
      y[(size_t)pix * C + c] = (op == ORC_POOL_AVERAGE) ? sum / (float)tally : best;
    }
  }
  return 0;
}

static inline int pool_equal(int op, float a, float b) {
  /* src/pooling/operators_impl.h:89-108 */
  if (a == b) return 1;
  return op == ORC_POOL_MAX_WITH_NAN && isnan(a) && isnan(b);
}

/* Max-pool gradient (src/pooling/kernels.h:142-243): dx[i] collects dy[o] from every
 * output o whose clamped window contains i, provided x[i] equals y[o] and no element
 * earlier in that window (row-major) also equals y[o].  x: forward input, y: forward
 * output, dy: incoming gradient (output-shaped), dx: result (input-shaped). */
int orc_pool_max_grad(int op, const float* x, const float* y, const float* dy, float* dx,
                      const OrcPoolParams* p) {
  const int C = p->channels;
  const long total = (long)p->batch * p->in_rows * p->in_cols;
#pragma omp parallel for schedule(static)
  for (long pix = 0; pix < total; ++pix) {
    const int w = (int)(pix % p->in_cols);
    const int h = (int)((pix / p->in_cols) % p->in_rows);
    const int n = (int)(pix / ((long)p->in_cols * p->in_rows));
    for (int c = 0; c < C; ++c) {
      const float xv = x[(size_t)pix * C + c];
      float grad = 0.f;
      for (int oh = 0; oh < p->out_rows; ++oh) {
        int r0 = oh * p->stride_rows - p->pad_rows;
        const int r1 = imin(r0 + p->window_rows, p->in_rows);
        r0 = imax(r0, 0);
        if (h < r0 || h >= r1) continue;
        for (int ow = 0; ow < p->out_cols; ++ow) {
          int c0 = ow * p->stride_cols - p->pad_cols;
          const int c1 = imin(c0 + p->window_cols, p->in_cols);
          c0 = imax(c0, 0);
          if (w < c0 || w >= c1) continue;
          const size_t o = (((size_t)n * p->out_rows + oh) * p->out_cols + ow) * C + c;
          const float yv = y[o];
          if (!pool_equal(op, xv, yv)) continue;
          int first = 1;
          for (int r = r0; r < r1 && first; ++r)
            for (int cc = c0; cc < c1; ++cc) {
              if (r == h && cc == w) { r = r1; break; }
              if (pool_equal(op, x[(((size_t)n * p->in_rows + r) * p->in_cols + cc) * C + c], yv)) {
                first = 0;
                break;
              }
            }
          if (first) grad += dy[o];
        }
      }
      dx[(size_t)pix * C + c] = grad;
    }
  }
  return 0;
}

/* Average-pool gradient (src/pooling/kernels.h:312-366): dx[i] = sum over outputs o
 * whose window contains i of dy[o] / valid_count(o), summed in float in (oh, ow) order. */
int orc_pool_avg_grad(const float* dy, float* dx, const OrcPoolParams* p) {
  const int C = p->channels;
  const long total = (long)p->batch * p->in_rows * p->in_cols;
#pragma omp parallel for schedule(static)
  for (long pix = 0; pix < total; ++pix) {
    const int w = (int)(pix % p->in_cols);
    const int h = (int)((pix / p->in_cols) % p->in_rows);
    const int n = (int)(pix / ((long)p->in_cols * p->in_rows));
    for (int c = 0; c < C; ++c) {
      float grad = 0.f;
      for (int oh = 0; oh < p->out_rows; ++oh) {
        int r0 = oh * p->stride_rows - p->pad_rows;
        const int r1 = imin(r0 + p->window_rows, p->in_rows);
        r0 = imax(r0, 0);
        if (h < r0 || h >= r1) continue;
        for (int ow = 0; ow < p->out_cols; ++ow) {
          int c0 = ow * p->stride_cols - p->pad_cols;
          const int c1 = imin(c0 + p->window_cols, p->in_cols);
          c0 = imax(c0, 0);
          if (w < c0 || w >= c1) continue;
          const int cnt = (r1 - r0) * (c1 - c0);
          grad += dy[(((size_t)n * p->out_rows + oh) * p->out_cols + ow) * C + c] / (float)cnt;
        }
      }
      dx[(size_t)pix * C + c] = grad;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* pointwise, bias, matmul, compat blend                                     */
/* ------------------------------------------------------------------------- */

/* relu = max(x,0), tanh, exp, log, floor, sqrt (src/pointwise/kernels.h:47-137). */
int orc_pointwise_forward(int op, const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const float v = x[i];
    switch (op) {
      case ORC_RELU: y[i] = fmaxf(v, 0.f); break;
      case ORC_TANH: y[i] = tanhf(v); break;
      case ORC_EXP: y[i] = expf(v); break;
      case ORC_LOG: y[i] = logf(v); break;
      case ORC_FLOOR: y[i] = floorf(v); break;
      case ORC_SQRT: y[i] = sqrtf(v); break;
      default: return 1;
    }
  }
  return 0;
}

/* The gradients as the reference's kernels compute them, with v the value handed in as the
 * first argument, which the kernel treats as the forward OUTPUT (src/pointwise/kernels.h:53-137,
 * 205-233): relu' = (v > 0 ? err : 0); tanh' = (1 - v*v) * err; log' = (1 / v) * err;
 * sqrt' = (0.5 / v) * err; exp' = exp(v) + err (sic: the reference marks it as to be corrected,
 * kernels.h:94-101).  Floor has no gradient. */
int orc_pointwise_grad(int op, const float* fwd, const float* err, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const float v = fwd[i], e = err[i];
    switch (op) {
      case ORC_RELU: out[i] = v > 0.f ? e : 0.f; break;
      case ORC_TANH: out[i] = (1.f - v * v) * e; break;
      case ORC_EXP: out[i] = expf(v) + e; break;
      case ORC_LOG: out[i] = (1.f / v) * e; break;
      case ORC_SQRT: out[i] = (0.5f / v) * e; break;
      default: return 1;
    }
  }
  return 0;
}

/* Binary operators with numpy-style broadcasting over at most four extents: the shorter shape is
 * padded with leading ones, each pair of extents must be equal or contain a one, and the output
 * takes the larger of each pair (include/portdnn/internal/binaryop/launch.h:34-57, 79-115; the
 * operators are src/binaryop/kernels.h Add / Sub / Mul / Div).  Returns 1 for shapes that cannot
 * be broadcast, more than four extents, an empty operand or an unknown operator. */
int orc_binaryop(int op, const float* lhs, const int* lhs_dims, int n_lhs, const float* rhs, const int* rhs_dims,
                 int n_rhs, float* out) {
  int ld[4] = {1, 1, 1, 1}, rd[4] = {1, 1, 1, 1}, od[4];
  if (n_lhs < 0 || n_lhs > 4 || n_rhs < 0 || n_rhs > 4 || op < 0 || op > 3) return 1;
  for (int i = 0; i < n_lhs; ++i) ld[4 - n_lhs + i] = lhs_dims[i];
  for (int i = 0; i < n_rhs; ++i) rd[4 - n_rhs + i] = rhs_dims[i];
  for (int i = 0; i < 4; ++i) {
    if (ld[i] <= 0 || rd[i] <= 0) return 1;
    if (ld[i] != rd[i] && ld[i] != 1 && rd[i] != 1) return 1;
    od[i] = ld[i] > rd[i] ? ld[i] : rd[i];
  }
  size_t o = 0;
  for (int a = 0; a < od[0]; ++a)
    for (int b = 0; b < od[1]; ++b)
      for (int c = 0; c < od[2]; ++c)
        for (int d = 0; d < od[3]; ++d, ++o) {
          const size_t li = (((size_t)(ld[0] == 1 ? 0 : a) * ld[1] + (ld[1] == 1 ? 0 : b)) * ld[2] +
                             (ld[2] == 1 ? 0 : c)) * ld[3] + (ld[3] == 1 ? 0 : d);
          const size_t ri = (((size_t)(rd[0] == 1 ? 0 : a) * rd[1] + (rd[1] == 1 ? 0 : b)) * rd[2] +
                             (rd[2] == 1 ? 0 : c)) * rd[3] + (rd[3] == 1 ? 0 : d);
          const float x = lhs[li], y = rhs[ri];
          out[o] = op == ORC_ADD ? x + y : op == ORC_SUB ? x - y : op == ORC_MUL ? x * y : x / y;
        }
  return 0;
}

/* out[i,c] = in[i,c] + bias[c]: binaryop Add with lhs_dims={rows,C}, rhs_dims={1,C}
 * (include/portdnn/binaryop/params.h:34-44, test/bias/bias_fixture.h:78-85). */
int orc_bias_add(const float* in, const float* bias, float* out, size_t rows, int C) {
  for (size_t i = 0; i < rows; ++i)
    for (int c = 0; c < C; ++c) out[i * C + c] = in[i * C + c] + bias[c];
  return 0;
}

/* out[b] = beta*out[b] + op(lhs[b]) * op(rhs[b]), row-major, strided batches
 * (include/portdnn/matmul/launch.h:37-39, src/matmul/kernels.h:34-127).
 * lhs is [m,k] ([k,m] if tl), rhs is [k,n] ([n,k] if tr).  Double accumulation. */
int orc_matmul(int tl, int tr, const float* lhs, const float* rhs, float* out, int batches, int m,
               int k, int n, float beta) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int b = 0; b < batches; ++b)
    for (int i = 0; i < m; ++i) {
      const float* A = lhs + (size_t)b * m * k;
      const float* B = rhs + (size_t)b * k * n;
      float* O = out + (size_t)b * m * n;
      for (int j = 0; j < n; ++j) {
        double acc = 0.0;
        for (int l = 0; l < k; ++l) {
          const double a = tl ? A[(size_t)l * m + i] : A[(size_t)i * k + l];
          const double bb = tr ? B[(size_t)j * k + l] : B[(size_t)l * n + j];
          acc += a * bb;
        }
        O[(size_t)i * n + j] = (beta == 0.f) ? (float)acc : (float)((double)beta * (double)O[(size_t)i * n + j] + acc);
      }
    }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* softmax, batchnorm (NHWC: `rows` pixels of C channels)                     */
/* ------------------------------------------------------------------------- */

/* y = exp(x - max_c x) / sum_c exp(x - max_c x) per pixel: the reference's five passes
 * (reduce Max, Sub, Exp, reduce Add, Div),
 * include/portdnn/internal/softmax/launch_internal.h:45-115. */
int orc_softmax_forward(const float* x, float* y, size_t rows, int C) {
  for (size_t i = 0; i < rows; ++i) {
    const float* xi = x + i * C;
    float* yi = y + i * C;
    float m = xi[0];
    for (int c = 1; c < C; ++c) m = fmaxf(m, xi[c]);
    float sum = 0.f;
    for (int c = 0; c < C; ++c) {
      yi[c] = expf(xi[c] - m);
      sum += yi[c];
    }
    for (int c = 0; c < C; ++c) yi[c] = yi[c] / sum;
  }
  return 0;
}

/* dx = (dy - sum_c(dy * y)) * y, with y the forward OUTPUT passed as `input`
 * (launch_internal.h:215-275: Mul, reduce Add, Sub, Mul). */
int orc_softmax_grad(const float* y, const float* dy, float* dx, size_t rows, int C) {
  for (size_t i = 0; i < rows; ++i) {
    float sum = 0.f;
    for (int c = 0; c < C; ++c) sum += dy[i * C + c] * y[i * C + c];
    for (int c = 0; c < C; ++c) dx[i * C + c] = (dy[i * C + c] - sum) * y[i * C + c];
  }
  return 0;
}

/* Batchnorm forward (include/portdnn/internal/batchnorm/launch_internal.h:95-158,187-310).
 * out = (x - mean) / sqrt(var + eps) * gamma + beta with the mean / variance HANDED IN, in both
 * modes.  Training additionally writes run_mean = batch_mean * (1 - m) + mean * m and
 * run_var = batch_var * (1 - m) + var * m, batch_var = mean((x - batch_mean)^2) (biased). */
int orc_batchnorm_forward(const float* x, const float* beta, const float* gamma, const float* mean,
                          const float* var, float* out, float* run_mean, float* run_var, size_t rows,
                          int C, float eps, float momentum, int training) {
  for (size_t i = 0; i < rows; ++i)
    for (int c = 0; c < C; ++c)
      out[i * C + c] = (x[i * C + c] - mean[c]) / sqrtf(var[c] + eps) * gamma[c] + beta[c];
  if (!training) return 0;
  for (int c = 0; c < C; ++c) {
    double sum = 0.0;
    for (size_t i = 0; i < rows; ++i) sum += x[i * C + c];
    const float bm = (float)(sum / (double)rows);
    double sq = 0.0;
    for (size_t i = 0; i < rows; ++i) {
      const float d = x[i * C + c] - bm;
      sq += (double)d * d;
    }
    const float bv = (float)(sq / (double)rows);
    run_mean[c] = bm * (1.f - momentum) + mean[c] * momentum;
    run_var[c] = bv * (1.f - momentum) + var[c] * momentum;
  }
  return 0;
}

/* Batchnorm gradient (launch_internal.h:318-535 training, 537-640 frozen).
 * Training: beta_grad = sum dy; with xc = x - batch_mean, v = batch_var + eps:
 *   gamma_grad = sum(dy * xc) / sqrt(v)
 *   out = ((dy - mean(dy)) - xc * (sum(dy * xc) / n / v)) * gamma / sqrt(v)
 * Frozen (population mean / variance handed in), s = sqrt(pop_var + eps):
 *   beta_grad = sum dy; gamma_grad = sum((x - pop_mean) * dy / s); out = dy * (gamma / s). */
int orc_batchnorm_grad(const float* x, const float* dy, const float* gamma, const float* pop_mean,
                       const float* pop_var, float* beta_grad, float* gamma_grad, float* out, size_t rows,
                       int C, float eps, int training) {
  for (int c = 0; c < C; ++c) {
    double sdy = 0.0;
    for (size_t i = 0; i < rows; ++i) sdy += dy[i * C + c];
    beta_grad[c] = (float)sdy;
    if (training) {
      double sx = 0.0;
      for (size_t i = 0; i < rows; ++i) sx += x[i * C + c];
      const float bm = (float)(sx / (double)rows);
      double sq = 0.0, sdx = 0.0;
      for (size_t i = 0; i < rows; ++i) {
        const float d = x[i * C + c] - bm;
        sq += (double)d * d;
        sdx += (double)dy[i * C + c] * d;
      }
      const float v = (float)(sq / (double)rows) + eps;
      const float sd = sqrtf(v);
      const float mean_dy = (float)sdy / (float)rows;
      const float k = (float)sdx / (float)rows / v;
      gamma_grad[c] = (float)sdx / sd;
      for (size_t i = 0; i < rows; ++i) {
        const float d = x[i * C + c] - bm;
        out[i * C + c] = ((dy[i * C + c] - mean_dy) - d * k) * gamma[c] / sd;
      }
    } else {
      const float sd = sqrtf(pop_var[c] + eps);
      double sg = 0.0;
      for (size_t i = 0; i < rows; ++i) sg += (double)((x[i * C + c] - pop_mean[c]) * dy[i * C + c] / sd);
      gamma_grad[c] = (float)sg;
      const float k = gamma[c] / sd;
      for (size_t i = 0; i < rows; ++i) out[i * C + c] = dy[i * C + c] * k;
    }
  }
  return 0;
}

/* TF-style padding (include/portdnn/helpers/padding.h:46-66): returns out size and
 * stores the low-side pad. */
int orc_padding(int in, int window, int stride, int same, int* pad_low) {
  if (same) {
    const int out = (in + stride - 1) / stride;
    const int need = (out - 1) * stride + window - in;
    *pad_low = need / 2;
    return out;
  }
  *pad_low = 0;
  const int num = in - window + 1;
  /* round_ratio_up (include/portdnn/helpers/ratio.h:43-49) */
  return num > 0 ? (num + stride - 1) / stride : num / stride;
}
