/*
 * CPU oracle for depthwise conv2d forward / backward-input / backward-filter.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * rosinality/depthwise-conv-pytorch (`torch_dwconv`) so that the CUDA library
 * can be checked against it.  Nothing in the shipped library links, loads or
 * calls it; only the test-suite, the smoke check and the CPU-baseline leg of
 * the benchmark do.
 *
 * Parity pin: the reference stores no golden vectors.  Its only CPU-executable
 * route is torch.nn.functional.conv2d(groups=C) (torch_dwconv/dwconv.py:125-128
 * and :166-173), which is also what its own tests compare against
 * (test/test_forward.py:14).  The fixtures under tests/golden/ were produced by
 * importing the reference package and running exactly those routes; this oracle
 * is checked against them in tests/test_oracle.py.
 *
 * Layout everywhere: contiguous NCHW activations, [C,1,kh,kw] filters.
 *
 * Two families:
 *   *_f64      direct sums in double: the numerical ground truth.
 *   *_f32seq   float arithmetic in the summation ORDER of the reference's
 *              kernels (row-major taps, one accumulator starting at zero, one
 *              fused multiply-add per tap; torch_dwconv/dwconv_kernel.cu:164-172
 *              and :403-429).  A CUDA kernel that keeps this order is
 *              bit-identical to these functions.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* Output extent of the reference's up/pad/correlate/decimate pipeline.
 * Follows make_conv2d_params, torch_dwconv/dwconv_kernel.cu:612-615. */
ORACLE_API int dwconv_oracle_out_size(int in, int up, int pad0, int pad1, int k,
                                      int down) {
  return (in * up + pad0 + pad1 - k + down) / down;
}

/* Small-map eligibility test of the reference.
 * Follows use_dwconv2d_small, torch_dwconv/dwconv_kernel.cu:652-662. */
ORACLE_API int dwconv_oracle_use_small(int in_h, int in_w, int kh, int kw,
                                       int up_h, int up_w, int down_h,
                                       int down_w, int pad_h, int pad_w) {
  int out_h = dwconv_oracle_out_size(in_h, up_h, pad_h, pad_h, kh, down_h);
  int out_w = dwconv_oracle_out_size(in_w, up_w, pad_w, pad_w, kw, down_w);
  return down_h == 1 && down_w == 1 && in_h <= 32 && in_w <= 32 &&
         in_h == out_h && in_w == out_w && pad_h >= 0 && pad_h < kh &&
         pad_w >= 0 && pad_w < kw && kh * kw <= (in_h + 1) / 2 * in_w;
}

ORACLE_API int dwconv_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------
 * fp64 ground truth
 * ---------------------------------------------------------------------- */

/* y[n,c,oy,ox] = sum_{ky,kx} x[n,c,oy*sh-ph+ky, ox*sw-pw+kx] * w[c,ky,kx]
 * (cross-correlation with zero padding: the forward direction of
 * dwconv2d_kernel, torch_dwconv/dwconv_kernel.cu:125-176 with up = 1). */
ORACLE_API void dwconv_oracle_forward_f64(const double *x, const double *w,
                                          double *y, int N, int C, int H, int W,
                                          int kh, int kw, int sh, int sw,
                                          int ph, int pw, int Ho, int Wo) {
  const long planes = (long)N * C;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < planes; ++nc) {
    const double *xp = x + nc * (long)H * W;
    const double *wp = w + (nc % C) * (long)kh * kw;
    double *yp = y + nc * (long)Ho * Wo;
    for (int oy = 0; oy < Ho; ++oy)
      for (int ox = 0; ox < Wo; ++ox) {
        double acc = 0.0;
        for (int ky = 0; ky < kh; ++ky) {
          int iy = oy * sh - ph + ky;
          if (iy < 0 || iy >= H) continue;
          for (int kx = 0; kx < kw; ++kx) {
            int ix = ox * sw - pw + kx;
            if (ix < 0 || ix >= W) continue;
            acc += xp[(long)iy * W + ix] * wp[ky * kw + kx];
          }
        }
        yp[(long)oy * Wo + ox] = acc;
      }
  }
}

/* dx[n,c,iy,ix] = sum over taps with (iy+ph-ky) % sh == 0 and
 * (ix+pw-kx) % sw == 0 of dy[n,c,(iy+ph-ky)/sh,(ix+pw-kx)/sw] * w[c,ky,kx].
 * The reference reaches the same values by zero-insertion upsampling of dy,
 * padding by (k-p-1, H-Ho*s+p) and correlating with the flipped filter
 * (torch_dwconv/dwconv.py:39-44,57-64; dwconv_kernel.cu:107-114). */
ORACLE_API void dwconv_oracle_backward_input_f64(
    const double *dy, const double *w, double *dx, int N, int C, int H, int W,
    int kh, int kw, int sh, int sw, int ph, int pw, int Ho, int Wo) {
  const long planes = (long)N * C;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < planes; ++nc) {
    const double *gp = dy + nc * (long)Ho * Wo;
    const double *wp = w + (nc % C) * (long)kh * kw;
    double *dp = dx + nc * (long)H * W;
    for (int iy = 0; iy < H; ++iy)
      for (int ix = 0; ix < W; ++ix) {
        double acc = 0.0;
        for (int ky = 0; ky < kh; ++ky) {
          int ny = iy + ph - ky;
          if (ny < 0 || ny % sh) continue;
          int oy = ny / sh;
          if (oy >= Ho) continue;
          for (int kx = 0; kx < kw; ++kx) {
            int nx = ix + pw - kx;
            if (nx < 0 || nx % sw) continue;
            int ox = nx / sw;
            if (ox >= Wo) continue;
            acc += gp[(long)oy * Wo + ox] * wp[ky * kw + kx];
          }
        }
        dp[(long)iy * W + ix] = acc;
      }
  }
}

/* dW[c,ky,kx] = sum_{n,oy,ox} dy[n,c,oy,ox] * x[n,c,oy*sh-ph+ky,ox*sw-pw+kx]
 * over in-range terms (dwconv2d_backward_kernel_kernel,
 * torch_dwconv/dwconv_kernel.cu:269-296). */
ORACLE_API void dwconv_oracle_backward_filter_f64(
    const double *x, const double *dy, double *dw, int N, int C, int H, int W,
    int kh, int kw, int sh, int sw, int ph, int pw, int Ho, int Wo) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    for (int ky = 0; ky < kh; ++ky)
      for (int kx = 0; kx < kw; ++kx) {
        double acc = 0.0;
        for (int n = 0; n < N; ++n) {
          const double *xp = x + ((long)n * C + c) * (long)H * W;
          const double *gp = dy + ((long)n * C + c) * (long)Ho * Wo;
          for (int oy = 0; oy < Ho; ++oy) {
            int iy = oy * sh - ph + ky;
            if (iy < 0 || iy >= H) continue;
            for (int ox = 0; ox < Wo; ++ox) {
              int ix = ox * sw - pw + kx;
              if (ix < 0 || ix >= W) continue;
              acc += gp[(long)oy * Wo + ox] * xp[(long)iy * W + ix];
            }
          }
        }
        dw[((long)c * kh + ky) * kw + kx] = acc;
      }
  }
}

static int floor_div_i(int a, int b) {
  int q = a / b;
  return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
}

/* The reference's general operator, as the extension exposes it
 * (dwconv2d, torch_dwconv/dwconv.cpp:27-35): zero-insert upsample by `up`,
 * pad by (pad0, pad1) (negative = crop), correlate with the filter (forward)
 * or with the filter flipped in both axes (backward;
 * dwconv_kernel.cu:107-114), keep every `down`-th sample.  Index algebra of
 * dwconv_kernel.cu:125-172: mid = out*down + up - 1 - pad0, in = floor(mid/up),
 * first tap = (in+1)*up - mid - 1, then taps step by `up`, inputs by 1.
 * Used to prove that forward/backward-input above are exactly the two ways
 * the reference's autograd function calls this operator. */
ORACLE_API void dwconv_oracle_upfirdn_f64(
    const double *in, const double *w, double *out, int N, int C, int in_h,
    int in_w, int kh, int kw, int up_y, int up_x, int down_y, int down_x,
    int pad_y0, int pad_y1, int pad_x0, int pad_x1, int forward) {
  const int out_h = dwconv_oracle_out_size(in_h, up_y, pad_y0, pad_y1, kh, down_y);
  const int out_w = dwconv_oracle_out_size(in_w, up_x, pad_x0, pad_x1, kw, down_x);
  const long planes = (long)N * C;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < planes; ++nc) {
    const double *ip = in + nc * (long)in_h * in_w;
    const double *wp = w + (nc % C) * (long)kh * kw;
    double *op = out + nc * (long)out_h * out_w;
    for (int oy = 0; oy < out_h; ++oy)
      for (int ox = 0; ox < out_w; ++ox) {
        int mid_y = oy * down_y + up_y - 1 - pad_y0;
        int mid_x = ox * down_x + up_x - 1 - pad_x0;
        int iy0 = floor_div_i(mid_y, up_y);
        int ix0 = floor_div_i(mid_x, up_x);
        int ty0 = (iy0 + 1) * up_y - mid_y - 1;
        int tx0 = (ix0 + 1) * up_x - mid_x - 1;
        double acc = 0.0;
        for (int ty = ty0, iy = iy0; ty < kh; ty += up_y, ++iy) {
          if (iy < 0 || iy >= in_h) continue;
          for (int tx = tx0, ix = ix0; tx < kw; tx += up_x, ++ix) {
            if (ix < 0 || ix >= in_w) continue;
            double tap = forward ? wp[ty * kw + tx]
                                 : wp[(kh - 1 - ty) * kw + (kw - 1 - tx)];
            acc += ip[(long)iy * in_w + ix] * tap;
          }
        }
        op[(long)oy * out_w + ox] = acc;
      }
  }
}

/* ------------------------------------------------------------------------
 * fp32 in the reference kernels' summation order
 * ---------------------------------------------------------------------- */

/* Forward, float: taps visited ky-major / kx-minor, padding taps contribute
 * fma(0, w, acc) (a no-op on the value), single accumulator from 0
 * (dwconv_kernel.cu:164-172). */
ORACLE_API void dwconv_oracle_forward_f32seq(const float *x, const float *w,
                                             float *y, int N, int C, int H,
                                             int W, int kh, int kw, int sh,
                                             int sw, int ph, int pw, int Ho,
                                             int Wo) {
  const long planes = (long)N * C;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < planes; ++nc) {
    const float *xp = x + nc * (long)H * W;
    const float *wp = w + (nc % C) * (long)kh * kw;
    float *yp = y + nc * (long)Ho * Wo;
    for (int oy = 0; oy < Ho; ++oy)
      for (int ox = 0; ox < Wo; ++ox) {
        float acc = 0.0f;
        for (int ky = 0; ky < kh; ++ky) {
          int iy = oy * sh - ph + ky;
          for (int kx = 0; kx < kw; ++kx) {
            int ix = ox * sw - pw + kx;
            float v = (iy >= 0 && iy < H && ix >= 0 && ix < W)
                          ? xp[(long)iy * W + ix]
                          : 0.0f;
            acc = fmaf(v, wp[ky * kw + kx], acc);
          }
        }
        yp[(long)oy * Wo + ox] = acc;
      }
  }
}

/* Backward-input, float, in the order the reference's flipped-filter
 * correlation visits the taps: flipped index t = k-1-ky ascending, i.e. ky
 * descending, and only taps of the matching stride phase
 * (dwconv_kernel.cu:107-114,150-172). */
ORACLE_API void dwconv_oracle_backward_input_f32seq(
    const float *dy, const float *w, float *dx, int N, int C, int H, int W,
    int kh, int kw, int sh, int sw, int ph, int pw, int Ho, int Wo) {
  const long planes = (long)N * C;
#pragma omp parallel for schedule(static)
  for (long nc = 0; nc < planes; ++nc) {
    const float *gp = dy + nc * (long)Ho * Wo;
    const float *wp = w + (nc % C) * (long)kh * kw;
    float *dp = dx + nc * (long)H * W;
    for (int iy = 0; iy < H; ++iy)
      for (int ix = 0; ix < W; ++ix) {
        float acc = 0.0f;
        for (int ky = kh - 1; ky >= 0; --ky) {
          int ny = iy + ph - ky;
          if (ny < 0 || ny % sh) continue;
          int oy = ny / sh;
          for (int kx = kw - 1; kx >= 0; --kx) {
            int nx = ix + pw - kx;
            if (nx < 0 || nx % sw) continue;
            int ox = nx / sw;
            float v = (oy < Ho && ox < Wo) ? gp[(long)oy * Wo + ox] : 0.0f;
            acc = fmaf(v, wp[ky * kw + kx], acc);
          }
        }
        dp[(long)iy * W + ix] = acc;
      }
  }
}
