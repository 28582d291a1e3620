/* CPU oracle for the Cu32 dense-contraction path.  TEST INFRASTRUCTURE ONLY: nothing in
 * the product library links, imports or calls this file; it exists so that tests, the smoke
 * check and the benchmark's CPU-baseline leg can check and time the reference's algorithm.
 *
 * Part 1 restates, loop for loop, the CPU check routines the reference uses to validate
 * its GPU kernels (they are the only CPU implementation of this path in the reference):
 *   multiply / multiplyT1 / multiplyT2   engine-cuda-base/Cuda_matMul/Cuda_matMul/test.cuh:60-82
 *   bmm / bmmT1 / bmmT2                  engine-cuda-base/Cuda_batchMatMul/Cuda_batchMatMul/test.cuh:97-140
 *   CONV_3D_NAIVE (float accumulator)    engine-cuda-base/Cuda_conv3D/Cuda_conv3D/test.cuh:171-200
 *   CONV_3D_img2col (double accumulator) engine-cuda-base/Cuda_conv3D/Cuda_conv3D/test.cuh:203-243
 *   samePercent (relative, thresholded)  Cuda_matMul/test.cuh:48-58, Cuda_conv3D/test.cuh:38-57,
 *                                        Cuda_batchMatMul/test.cuh:69-89
 *   buf_summary (Kahan)                  Cuda_matMul/Cuda_matMul/SKbufsum.cuh:29-68
 *   filter remode W[OC,FH,FW,IC] -> CW[FH,FW,IC,OC]   Cuda_conv3D/conv3D_kernel_remode_V1.cuh:50-196
 *   deconv3D_deltaX_img2col_s1 (float accumulator)   engine-cuda-base/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/test.cuh:154-196
 *   deconv3D_deltaX_img2col (any stride)             same file, :109-152
 *   ks_remode / ks_remodev2 (filter workspace of the strided data gradient; GPU kernels, restated element by
 *   element)                                         dconv3D_dX_kernelSplit_remode_v1.cuh:28-66, _v2.cuh:31-66
 *   linear2D (y = alpha*x + beta, the attention block's scale; a GPU kernel)   Cuda_function/type1_linear2D.cuh:40-58
 *   softmax2D (the engine's row softmax: row_max, row_softmax, div2D_field; GPU kernels, restated row by row - the
 *   arithmetic per element is theirs, the order of the row sum is not: the kernels sum strided partial sums with
 *   Kahan compensation through a tree, here one compensated sum runs along the row, so the results agree to a
 *   few units in the last place and are pinned on the GPU with that tolerance)
 *                                                    Cuda_reduce/row_max.cuh:60-105, row_softmax.cuh:45-120,
 *                                                    Cuda_function/type1_div2D_field.cuh:42-68
 *   deconv3d_deltaW_naive (the Java check loop of the weight gradient; PARITY UNPINNED, see below)
 *                                                    ZUTIL-STD-1.2/src/z/util/math/vector/Tense.java:1276-1318
 *   linear_dual2D_row (the bias-row add the engine applies right after matMul / conv3D;
 *   a GPU kernel, restated element by element)        Cuda_function/Cuda_function/type1_linear_dual2D_row.cuh:41-70
 * Loop order and accumulation type follow the reference exactly (k outermost, FP32 "+=" into
 * C), so that on the same inputs the results are bit-identical to the reference routines
 * compiled with the same compiler flags; oracle/build_ref.py builds those routines from the
 * reference tree and tests/test_oracle.py checks the identity.
 *
 * Part 2 holds FP64-accumulating versions of the same contractions; they are the accuracy
 * oracle the GPU results are measured against.
 *
 * Pinning status: pinned against the reference's own routines compiled here (see above) and
 * against hand-computed known answers in tests/golden/; the reference ships no golden vectors.
 * Exception - parity unpinned: the weight-gradient loop.  The reference publishes no CUDA source for
 * Cuda_dconv3D_deltaW and its only CPU statement of it is Java, which cannot be run here; the restatement is checked
 * against the FP64 version, and that against the pinned forward-convolution oracle (tests/test_deltaw.py).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/* ------------------------------------------------------------------ part 1: reference loops */

/* C[N,M] += A[N,K] * B[K,M]   (caller zeroes C first, as the reference's newPtr does) */
void oracle_multiply(const float* A, const float* B, float* C, int N, int M, int K) {
  for (int k = 0; k < K; k++)
    for (int i = 0; i < N; i++)
      for (int j = 0; j < M; j++)
        C[(size_t)i * M + j] += A[(size_t)i * K + k] * B[(size_t)k * M + j];
}

/* C[N,M] += A[K,N]^T * B[K,M] */
void oracle_multiplyT1(const float* A, const float* B, float* C, int N, int M, int K) {
  for (int k = 0; k < K; k++)
    for (int i = 0; i < N; i++)
      for (int j = 0; j < M; j++)
        C[(size_t)i * M + j] += A[(size_t)k * N + i] * B[(size_t)k * M + j];
}

/* C[N,M] += A[N,K] * B[M,K]^T */
void oracle_multiplyT2(const float* A, const float* B, float* C, int N, int M, int K) {
  for (int k = 0; k < K; k++)
    for (int i = 0; i < N; i++)
      for (int j = 0; j < M; j++)
        C[(size_t)i * M + j] += A[(size_t)i * K + k] * B[(size_t)j * K + k];
}

/* C[b][N,CM] += A[b][N,AK] * B[b][BK,CM], reduction over BK */
void oracle_bmm(const float* A, const float* B, float* C, int Batch, int N, int CM, int BK, int AK) {
  for (int b = 0; b < Batch; b++)
    for (int k = 0; k < BK; k++)
      for (int i = 0; i < N; i++)
        for (int j = 0; j < CM; j++)
          C[((size_t)b * N + i) * CM + j] +=
              A[((size_t)b * N + i) * AK + k] * B[((size_t)b * BK + k) * CM + j];
}

/* C[b][CN,CM] += A[b][K,AN]^T * B[b][K,CM] */
void oracle_bmmT1(const float* A, const float* B, float* C, int Batch, int CN, int AN, int CM, int K) {
  for (int b = 0; b < Batch; b++)
    for (int k = 0; k < K; k++)
      for (int i = 0; i < CN; i++)
        for (int j = 0; j < CM; j++)
          C[((size_t)b * CN + i) * CM + j] +=
              A[((size_t)b * K + k) * AN + i] * B[((size_t)b * K + k) * CM + j];
}

/* C[b][N,CM] (columns < BM) += A[b][N,K] * B[b][BM,K]^T */
void oracle_bmmT2(const float* A, const float* B, float* C, int Batch, int N, int CM, int BM, int K) {
  for (int b = 0; b < Batch; b++)
    for (int k = 0; k < K; k++)
      for (int i = 0; i < N; i++)
        for (int j = 0; j < BM; j++)
          C[((size_t)b * N + i) * CM + j] +=
              A[((size_t)b * N + i) * K + k] * B[((size_t)b * BM + j) * K + k];
}

#define X4(n, h, w, c) X[(((size_t)(n) * IH + (h)) * IW + (w)) * IC + (c)]
#define W4(o, h, w, c) W[(((size_t)(o) * FH + (h)) * FW + (w)) * IC + (c)]
#define Y4(n, h, w, c) Y[(((size_t)(n) * OH + (h)) * OW + (w)) * OC + (c)]

/* Direct convolution, FP32 accumulator, taps outside the image skipped. */
void oracle_conv3D_naive(const float* X, int IH, int IW, const float* W, int FH, int FW, float* Y,
                         int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  for (int oc = 0; oc < OC; oc++)
    for (int n = 0; n < N; n++) {
      int ih_s, iw_s, oh, ow;
      for (ih_s = -ph, oh = 0; ih_s <= (IH + ph - FH); ih_s += sh, oh++)
        for (iw_s = -pw, ow = 0; iw_s <= (IW + pw - FW); iw_s += sw, ow++) {
          float v = 0;
          for (int fh = 0; fh < FH; fh++)
            for (int fw = 0; fw < FW; fw++)
              for (int ic = 0; ic < IC; ic++) {
                int ih = ih_s + fh, iw = iw_s + fw;
                if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                v += X4(n, ih, iw, ic) * W4(oc, fh, fw, ic);
              }
          Y4(n, oh, ow, oc) = v;
        }
    }
}

/* The same convolution walked as the implicit GEMM (GN = OC, GM = N*OH*OW, GK = FH*FW*IC)
 * with a double accumulator. */
void oracle_conv3D_img2col(const float* X, int IH, int IW, const float* W, int FH, int FW, float* Y,
                           int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  int GN = OC, GM = N * OH * OW, GK = FH * FW * IC;
  for (int i = 0; i < GN; i++) {
    int oc = i;
    for (int j = 0; j < GM; j++) {
      int n = j / (OH * OW), j_res = j % (OH * OW);
      int oh = j_res / OW, ow = j_res % OW;
      double v = 0;
      for (int k = 0; k < GK; k++) {
        int fh = k / (FW * IC), k_res = k % (FW * IC);
        int fw = k_res / IC, ic = k_res % IC;
        int ih = oh * sh - ph + fh, iw = ow * sw - pw + fw;
        if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
        v += X4(n, ih, iw, ic) * W4(oc, fh, fw, ic);
      }
      Y4(n, oh, ow, oc) = (float)v;
    }
  }
}

/* Fraction of elements with |a-b| / |a+b| < threshold (equal elements count as same). */
float oracle_samePercent_relative(const float* a, const float* b, int length, float threshold) {
  int sum = 0;
  for (int i = 0; i < length; i++) {
    if (a[i] == b[i]) { sum++; continue; }
    float dif = fabsf((a[i] - b[i]) / (a[i] + b[i]));
    if (dif < threshold) sum++;
  }
  return 1.0f * sum / length;
}

/* Fraction of elements with |a-b| < threshold (the batched tests' absolute criterion). */
float oracle_samePercent_absolute(const float* a, const float* b, int length, float threshold) {
  int sum = 0;
  for (int i = 0; i < length; i++) {
    if (a[i] == b[i]) { sum++; continue; }
    if (fabsf(a[i] - b[i]) < threshold) sum++;
  }
  return 1.0f * sum / length;
}

float oracle_zeroPercent(const float* a, int length) {
  int sum = 0;
  for (int i = 0; i < length; i++)
    if (a[i] == 0) sum++;
  return 1.0f * sum / length;
}

/* C += sum_p Cbuf[p], Kahan-compensated in FP32, element by element. */
void oracle_buf_summary(const float* Cbuf, float* C, int part, int sizeC) {
  for (int i = 0; i < sizeC; i++) {
    volatile float v = C[i], c = 0.0f;
    for (int p = 0; p < part; p++) {
      volatile float vbuf = Cbuf[(size_t)p * sizeC + i];
      vbuf -= c;
      volatile float t = v + vbuf;
      volatile float d = t - v;
      c = d - vbuf;
      v = t;
    }
    C[i] = v;
  }
}

/* Data gradient of the stride-1 convolution, the reference's check loop: for every input pixel and
 * channel, a float accumulator over k = (oc, fh, fw) in that order, the filter applied rotated:
 * deltaX[n,ih,iw,ic] = sum deltaY[n, ih-(FH-1-ph)+fh, iw-(FW-1-pw)+fw, oc] * W[oc, FH-1-fh, FW-1-fw, ic]. */
void oracle_deconv3D_deltaX_img2col_s1(const float* deltaY, int OH, int OW, const float* W, int FH, int FW,
                                       float* deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  const int oph = FH - ph - 1, opw = FW - pw - 1;
  const int GK = OC * FH * FW;
  for (int ic = 0; ic < IC; ic++)
    for (int j = 0; j < N * IH * IW; j++) {
      const int n = j / (IH * IW), jr = j % (IH * IW);
      const int ih = jr / IW, iw = jr % IW;
      float v = 0;
      for (int k = 0; k < GK; k++) {
        const int oc = k / (FH * FW), kr = k % (FH * FW);
        const int fh = kr / FW, fw = kr % FW;
        const int oh = ih - oph + fh, ow = iw - opw + fw;
        if (oh < 0 || ow < 0 || oh >= OH || ow >= OW) continue;
        v += deltaY[(((size_t)n * OH + oh) * OW + ow) * OC + oc] *
             W[(((size_t)oc * FH + (FH - 1 - fh)) * FW + (FW - 1 - fw)) * IC + ic];
      }
      deltaX[(((size_t)n * IH + ih) * IW + iw) * IC + ic] = v;
    }
}

/* Any stride, the reference's check loop: deltaY is thought of as dilated by the stride (OH_p rows), the rotated
 * filter walks it, positions that fall between the dilated pixels are skipped; float accumulator, k = (oc, fh, fw). */
void oracle_deconv3D_deltaX_img2col(const float* deltaY, int OH, int OW, const float* W, int FH, int FW,
                                    float* deltaX, int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph,
                                    int pw) {
  const int OH_p = OH + (OH - 1) * (sh - 1), OW_p = OW + (OW - 1) * (sw - 1);
  const int oph = FH - ph - 1, opw = FW - pw - 1;
  const int GK = OC * FH * FW;
  for (int ic = 0; ic < IC; ic++)
    for (int j = 0; j < N * IH * IW; j++) {
      const int n = j / (IH * IW), jr = j % (IH * IW);
      const int ih = jr / IW, iw = jr % IW;
      float v = 0;
      for (int k = 0; k < GK; k++) {
        const int oc = k / (FH * FW), kr = k % (FH * FW);
        const int fh = kr / FW, fw = kr % FW;
        const int oh = ih - oph + fh, ow = iw - opw + fw;
        if (oh < 0 || ow < 0 || oh >= OH_p || ow >= OW_p) continue;
        if (oh % sh != 0 || ow % sw != 0) continue;
        v += deltaY[(((size_t)n * OH + oh / sh) * OW + ow / sw) * OC + oc] *
             W[(((size_t)oc * FH + (FH - 1 - fh)) * FW + (FW - 1 - fw)) * IC + ic];
      }
      deltaX[(((size_t)n * IH + ih) * IW + iw) * IC + ic] = v;
    }
}

/* Any stride with an FP64 accumulator: every deltaY pixel scatters into the input positions it was computed from. */
void oracle_deconv3D_deltaX_f64(const float* deltaY, int OH, int OW, const float* W, int FH, int FW, double* deltaX,
                                int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  for (size_t i = 0; i < (size_t)N * IH * IW * IC; i++) deltaX[i] = 0.0;
  for (int n = 0; n < N; n++)
    for (int oh = 0; oh < OH; oh++)
      for (int ow = 0; ow < OW; ow++) {
        const float* dy = deltaY + (((size_t)n * OH + oh) * OW + ow) * OC;
        for (int fh = 0; fh < FH; fh++) {
          const int ih = oh * sh - ph + fh;
          if (ih < 0 || ih >= IH) continue;
          for (int fw = 0; fw < FW; fw++) {
            const int iw = ow * sw - pw + fw;
            if (iw < 0 || iw >= IW) continue;
            double* out = deltaX + (((size_t)n * IH + ih) * IW + iw) * IC;
            for (int oc = 0; oc < OC; oc++) {
              const float* w = W + (((size_t)oc * FH + fh) * FW + fw) * IC;
              const double d = dy[oc];
              for (int ic = 0; ic < IC; ic++) out[ic] += d * (double)w[ic];
            }
          }
        }
      }
}

/* Filter workspace of the strided data gradient.  v2 != 0: CW[y][x][fhr][fwr][oc][ic]; v2 == 0: CW[y][x][oc][fhr][fwr][ic];
 * tap (fhr, fwr) of phase (y, x) is W[oc][y + (CFH_y-1-fhr)*sh][x + (CFW_x-1-fwr)*sw][ic]; each phase starts at a slot
 * of OC*mCFH*mCFW*IC floats and fills only its own OC*CFH_y*CFW_x*IC; the rest of CW is left as it was. */
void oracle_ks_remode(int v2, const float* W, int FH, int FW, float* CW, int mCFH, int mCFW, int OC, int IC, int sh,
                      int sw) {
  for (int by = 0; by < sh * sw; by++) {
    float* cw = CW + (size_t)by * OC * mCFH * mCFW * IC;
    const int y = by / sw, x = by - y * sw;
    const int CFH = (FH - y + sh - 1) / sh, CFW = (FW - x + sw - 1) / sw;
    if (CFH <= 0 || CFW <= 0) continue;
    for (int oc = 0; oc < OC; oc++)
      for (int fhr = 0; fhr < CFH; fhr++)
        for (int fwr = 0; fwr < CFW; fwr++)
          for (int ic = 0; ic < IC; ic++) {
            const int fh = y + (CFH - 1 - fhr) * sh, fw = x + (CFW - 1 - fwr) * sw;
            const float w = (fh < FH && fw < FW) ? W[(((size_t)oc * FH + fh) * FW + fw) * IC + ic] : 0.0f;
            const size_t idx = v2 ? ((((size_t)fhr * CFW + fwr) * OC + oc) * IC + ic)
                                  : ((((size_t)oc * CFH + fhr) * CFW + fwr) * IC + ic);
            cw[idx] = w;
          }
  }
}

/* The same gradient with an FP64 accumulator (accuracy oracle). */
void oracle_deconv3D_deltaX_s1_f64(const float* deltaY, int OH, int OW, const float* W, int FH, int FW,
                                   double* deltaX, int IH, int IW, int N, int IC, int OC, int ph, int pw) {
  for (int n = 0; n < N; n++)
    for (int ih = 0; ih < IH; ih++)
      for (int iw = 0; iw < IW; iw++) {
        double* out = deltaX + (((size_t)n * IH + ih) * IW + iw) * IC;
        for (int ic = 0; ic < IC; ic++) out[ic] = 0.0;
        for (int fh = 0; fh < FH; fh++) {
          const int oh = ih + ph - fh;
          if (oh < 0 || oh >= OH) continue;
          for (int fw = 0; fw < FW; fw++) {
            const int ow = iw + pw - fw;
            if (ow < 0 || ow >= OW) continue;
            const float* dy = deltaY + (((size_t)n * OH + oh) * OW + ow) * OC;
            for (int oc = 0; oc < OC; oc++) {
              const float* w = W + (((size_t)oc * FH + fh) * FW + fw) * IC;
              const double d = dy[oc];
              for (int ic = 0; ic < IC; ic++) out[ic] += d * (double)w[ic];
            }
          }
        }
      }
}

/* Y[i] = alpha*X1[i] + beta*X2[i % row_lengthv] + gamma for every element of the padded
 * [height][stride] matrix, then zero where the column (i % stride) is at or beyond width.
 * With the coefficients the engine uses for a bias add (1, 1, 0) every product is exact and
 * the result is the single rounding of X1 + X2, whatever the contraction into FMAs. */
void oracle_linear_dual2D_row(const float* X1, const float* X2, int row_lengthv, float alpha, float beta,
                              float gamma, float* Y, int lengthv, int width, int stride) {
  for (int i = 0; i < lengthv; i++) {
    volatile float a = alpha * X1[i];
    volatile float b = beta * X2[i % row_lengthv];
    volatile float y = a + b;
    y = y + gamma;
    Y[i] = ((i % stride) < width) ? y : 0.0f;
  }
}

/* CW[fh,fw,ic,oc] = W[oc,fh,fw,ic] */
void oracle_kernel_remode(const float* W, float* CW, int FH, int FW, int OC, int IC) {
  size_t G = (size_t)FH * FW * IC;
  for (int oc = 0; oc < OC; oc++)
    for (size_t g = 0; g < G; g++) CW[g * OC + oc] = W[(size_t)oc * G + g];
}

/* ------------------------------------------------------------------ part 2: FP64 oracle */

/* Row-range versions so callers can run slices on several host threads. */
void oracle_multiply_f64(const float* A, const float* B, double* C, int N, int M, int K, int form,
                         int row_begin, int row_end) {
  /* form 0: A[N,K] B[K,M]; 1: A[K,N]^T B[K,M]; 2: A[N,K] B[M,K]^T.  C is [N,M] doubles. */
  for (int i = row_begin; i < row_end; i++) {
    double* c = C + (size_t)i * M;
    for (int j = 0; j < M; j++) c[j] = 0.0;
    for (int k = 0; k < K; k++) {
      double a = form == 1 ? (double)A[(size_t)k * N + i] : (double)A[(size_t)i * K + k];
      if (form == 2) {
        for (int j = 0; j < M; j++) c[j] += a * (double)B[(size_t)j * K + k];
      } else {
        const float* b = B + (size_t)k * M;
        for (int j = 0; j < M; j++) c[j] += a * (double)b[j];
      }
    }
  }
}

void oracle_conv3D_f64(const float* X, int IH, int IW, const float* W, int FH, int FW, double* Y,
                       int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                       int n_begin, int n_end) {
  for (int n = n_begin; n < n_end; n++)
    for (int oh = 0; oh < OH; oh++)
      for (int ow = 0; ow < OW; ow++)
        for (int oc = 0; oc < OC; oc++) {
          double v = 0.0;
          for (int fh = 0; fh < FH; fh++) {
            int ih = oh * sh - ph + fh;
            if (ih < 0 || ih >= IH) continue;
            for (int fw = 0; fw < FW; fw++) {
              int iw = ow * sw - pw + fw;
              if (iw < 0 || iw >= IW) continue;
              const float* x = &X4(n, ih, iw, 0);
              const float* w = &W4(oc, fh, fw, 0);
              for (int ic = 0; ic < IC; ic++) v += (double)x[ic] * (double)w[ic];
            }
          }
          Y[(((size_t)n * OH + oh) * OW + ow) * OC + oc] = v;
        }
}

/* ------------------------------------------------------------------ weight gradient of the convolution
 * The reference's CUDA source for Cuda_dconv3D_deltaW is not published; its Java test
 * (test/cuda/conv3D/Cuda_conv3D_dW_test.java:64-98) checks the natives against Tense.deconv3d_deltaW_naive
 * (ZUTIL-STD-1.2/src/z/util/math/vector/Tense.java:1276-1318), which swaps the N and IC axes of X, spreads deltaY
 * over a zero-dilated OHp x OWp grid and calls Tense.conv3D_naive (:same file; FP32 products summed in a double,
 * loops over grid rows, grid columns, then images).  Restated here without the temporaries: the dilated grid's zero
 * entries add 0.0 to the sum, so only the live positions are visited, in the same order. */
void oracle_deconv3D_deltaW_naive(const float* X, int IH, int IW, const float* deltaY, int OH, int OW, float* deltaW,
                                  int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  for (int ic = 0; ic < IC; ic++)
    for (int oc = 0; oc < OC; oc++)
      for (int fh = 0; fh < FH; fh++)
        for (int fw = 0; fw < FW; fw++) {
          double v = 0;
          for (int oh = 0; oh < OH; oh++) {
            const int ih = fh - ph + oh * sh;
            if (ih < 0 || ih >= IH) continue;
            for (int ow = 0; ow < OW; ow++) {
              const int iw = fw - pw + ow * sw;
              if (iw < 0 || iw >= IW) continue;
              for (int n = 0; n < N; n++) {
                const float prod = X[(((size_t)n * IH + ih) * IW + iw) * IC + ic] *
                                   deltaY[(((size_t)n * OH + oh) * OW + ow) * OC + oc];
                v += prod;
              }
            }
          }
          deltaW[(((size_t)oc * FH + fh) * FW + fw) * IC + ic] = (float)v;
        }
}

/* FP64 throughout (exact products of FP32 inputs, double accumulator). */
void oracle_deconv3D_deltaW_f64(const float* X, int IH, int IW, const float* deltaY, int OH, int OW, double* deltaW,
                                int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw) {
  for (size_t i = 0; i < (size_t)OC * FH * FW * IC; i++) deltaW[i] = 0.0;
  for (int n = 0; n < N; n++)
    for (int oh = 0; oh < OH; oh++)
      for (int ow = 0; ow < OW; ow++) {
        const float* dy = deltaY + (((size_t)n * OH + oh) * OW + ow) * OC;
        for (int fh = 0; fh < FH; fh++) {
          const int ih = oh * sh - ph + fh;
          if (ih < 0 || ih >= IH) continue;
          for (int fw = 0; fw < FW; fw++) {
            const int iw = ow * sw - pw + fw;
            if (iw < 0 || iw >= IW) continue;
            const float* x = X + (((size_t)n * IH + ih) * IW + iw) * IC;
            for (int oc = 0; oc < OC; oc++) {
              double* out = deltaW + (((size_t)oc * FH + fh) * FW + fw) * IC;
              const double d = dy[oc];
              for (int ic = 0; ic < IC; ic++) out[ic] += d * (double)x[ic];
            }
          }
        }
      }
}

/* Y = alpha * X + beta, element by element: the reference's linear2D kernel (Cuda_function/type1_linear2D.cuh:40-58
 * with simdLinear4, micro.cuh:54-58: x * alpha + beta, which nvcc contracts to one fused multiply-add). */
void oracle_linear2D(float alpha, const float* X, float beta, float* Y, long long length) {
  for (long long i = 0; i < length; i++) Y[i] = fmaf(X[i], alpha, beta);
}

/* Row softmax as the engine's softmax2D computes it (CudaFloat32EngineBase.java:5738-5775):
 *   row_max      m = max over the whole row of `stride` floats, pitch padding included (row_max.cuh:60-105)
 *   row_softmax  e = expf(x - m), zero beyond `width`; V = sum of e, Kahan-compensated, four elements per step
 *                (row_softmax.cuh:62-75, micro.cuh:170-174)
 *   div2D_field  y = e * (1 / V) + 0, zero beyond `width` (type1_div2D_field.cuh:42-68 with alpha = 1, beta = gamma = 0)
 * stride is a multiple of 4. */
void oracle_softmax2D(const float* X, float* Y, long long rows, int stride, int width) {
    for (long long r = 0; r < rows; ++r) {
        const float* x = X + r * stride;
        float* y = Y + r * stride;
        float m = -3.402823466e+38f;
        for (int c = 0; c < stride; ++c) m = fmaxf(m, x[c]);
        float v = 0.0f, comp = 0.0f;
        for (int c = 0; c < stride; c += 4) {
            float e[4];
            for (int j = 0; j < 4; ++j) {
                e[j] = expf(x[c + j] - m);
                e[j] *= (float)((c + j) % stride < width);
                y[c + j] = e[j];
            }
            const float dv = (e[0] + e[1] + e[2] + e[3]) - comp;
            const float t = v + dv;
            comp = (t - v) - dv;
            v = t;
        }
        const float rv = 1.0f / (1.0f * v + 0.0f);
        for (int c = 0; c < stride; ++c) y[c] = (c < width) ? (y[c] * rv + 0.0f) : 0.0f;
    }
}
