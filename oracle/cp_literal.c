/* Literal CPU restatement of the reference's CP4 conv2d loops, in plain C.
 * TEST INFRASTRUCTURE ONLY: it is the checker for small cases and (for the
 * forward) one leg of the timed CPU baseline; the shipped library never links it.
 *
 * Arithmetic is fp32 in the reference's own accumulation order wherever that
 * order is sequential in the reference:
 *   cp4lit_forward        : Cuda_kernels/cp4Conv2dForward.cu:84-133 (one channel lane)
 *   cp4lit_backward_data  : Cuda_kernels/cp4Conv2dBackwardData.cu:57-108
 *   cp4lit_backward_filter_{t,c,y,x,full} :
 *                           Cuda_kernels/cp4Conv2dBackwardFilter.cu:91-104,142-155,192-205,241-254,47-56
 * Layouts: In [N,C,H,W], Out [N,T,H,W], FT [T,R], FC [C,R], FY [Y,R], FX [X,R], row-major.
 * Out-of-range reads are zero (the reference reads a zero-padded copy).
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -o oracle/_build/libcp_literal.so oracle/cp_literal.c
 */
#include <stdlib.h>
#include <string.h>

typedef struct {
  unsigned N, H, W, pad, T, C, Y, X, Rank;
} cp4lit_shape;

static inline float in_at(const float* In, const cp4lit_shape* s, unsigned nch, unsigned n, unsigned c, long h, long w) {
  if (h < 0 || w < 0 || h >= (long)s->H || w >= (long)s->W) return 0.0f;
  return In[(((size_t)n * nch + c) * s->H + (size_t)h) * s->W + (size_t)w];
}

/* Forward.  The reference strides channels over Bc lanes and tree-reduces the
 * lanes; with Bc = 1 (chosen for C < 32) the order below is the kernel's. */
void cp4lit_forward(const cp4lit_shape* s, const float* In, const float* FT, const float* FC, const float* FY,
                    const float* FX, float* Out) {
  const unsigned R = s->Rank;
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned n = 0; n < s->N; ++n)
    for (unsigned h = 0; h < s->H; ++h) {
      float* c_acc = (float*)malloc(sizeof(float) * R * 2);
      float* pix_acc = c_acc + R;
      for (unsigned w = 0; w < s->W; ++w) {
        for (unsigned r = 0; r < R; ++r) c_acc[r] = 0.0f;
        for (unsigned c = 0; c < s->C; ++c) {
          for (unsigned r = 0; r < R; ++r) pix_acc[r] = 0.0f;
          for (unsigned y = 0; y < s->Y; ++y)
            for (unsigned x = 0; x < s->X; ++x) {
              const long hh = (long)h + y - s->pad, ww = (long)w + x - s->pad;
              if (hh < 0 || ww < 0 || hh >= (long)s->H || ww >= (long)s->W) continue;
              const float v = In[(((size_t)n * s->C + c) * s->H + hh) * s->W + ww];
              for (unsigned r = 0; r < R; ++r) pix_acc[r] += v * FY[y * R + r] * FX[x * R + r];
            }
          for (unsigned r = 0; r < R; ++r) c_acc[r] += pix_acc[r] * FC[c * R + r];
        }
        for (unsigned t = 0; t < s->T; ++t) {
          float out_acc = 0.0f;
          for (unsigned r = 0; r < R; ++r) out_acc += c_acc[r] * FT[t * R + r];
          Out[(((size_t)n * s->T + t) * s->H + h) * s->W + w] = out_acc;
        }
      }
      free(c_acc);
    }
}

/* Backward data: In is the upstream gradient [N,T,H,W], Out is [N,C,H,W]. */
void cp4lit_backward_data(const cp4lit_shape* s, const float* In, const float* FT, const float* FC, const float* FY,
                          const float* FX, float* Out) {
  const unsigned R = s->Rank;
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned n = 0; n < s->N; ++n)
    for (unsigned h = 0; h < s->H; ++h) {
      float* acc = (float*)malloc(sizeof(float) * R * 2);
      float* tmpxl = acc + R;
      for (unsigned w = 0; w < s->W; ++w) {
        for (unsigned r = 0; r < R; ++r) acc[r] = 0.0f;
        for (unsigned t = 0; t < s->T; ++t) {
          for (unsigned r = 0; r < R; ++r) tmpxl[r] = 0.0f;
          for (unsigned y = 0; y < s->Y; ++y)
            for (unsigned x = 0; x < s->X; ++x) {
              const float v = in_at(In, s, s->T, n, t, (long)h + y - s->pad, (long)w + x - s->pad);
              for (unsigned r = 0; r < R; ++r)
                tmpxl[r] += v * FY[(s->Y - 1 - y) * R + r] * FX[(s->X - 1 - x) * R + r];
            }
          for (unsigned r = 0; r < R; ++r) acc[r] += tmpxl[r] * FT[t * R + r];
        }
        for (unsigned c = 0; c < s->C; ++c) {
          float v = 0.0f;
          for (unsigned r = 0; r < R; ++r) v += acc[r] * FC[c * R + r];
          Out[(((size_t)n * s->C + c) * s->H + h) * s->W + w] = v;
        }
      }
      free(acc);
    }
}

static float* padded_copy(const cp4lit_shape* s, const float* In) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad;
  float* P = (float*)calloc((size_t)s->N * s->C * sH * sW, sizeof(float));
  for (unsigned n = 0; n < s->N; ++n)
    for (unsigned c = 0; c < s->C; ++c)
      for (unsigned h = 0; h < s->H; ++h)
        memcpy(P + (((size_t)n * s->C + c) * sH + h + s->pad) * sW + s->pad,
               In + (((size_t)n * s->C + c) * s->H + h) * s->W, sizeof(float) * s->W);
  return P;
}

#define DLDO(n, t, h, w) dLdO[(((size_t)(n) * s->T + (t)) * s->H + (h)) * s->W + (w)]
#define SHIN(n, c, h, w) SHIn[(((size_t)(n) * s->C + (c)) * sH + (h)) * sW + (w)]

/* The four nests accumulate with += into a caller-zeroed gradient, in the
 * reference's loop order, one fp32 accumulator per gradient element. */
void cp4lit_backward_filter_t(const cp4lit_shape* s, float* dFT, const float* In, const float* dLdO, const float* FC,
                              const float* FY, const float* FX) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad, R = s->Rank;
  float* SHIn = padded_copy(s, In);
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned t = 0; t < s->T; ++t)
    for (unsigned r = 0; r < R; ++r) {
      float a = dFT[t * R + r];
      for (unsigned n = 0; n < s->N; ++n)
        for (unsigned h = 0; h < s->H; ++h)
          for (unsigned w = 0; w < s->W; ++w)
            for (unsigned c = 0; c < s->C; ++c)
              for (unsigned y = 0; y < s->Y; ++y)
                for (unsigned x = 0; x < s->X; ++x)
                  a += DLDO(n, t, h, w) * SHIN(n, c, h + y, w + x) * FC[c * R + r] * FY[y * R + r] * FX[x * R + r];
      dFT[t * R + r] = a;
    }
  free(SHIn);
}

void cp4lit_backward_filter_c(const cp4lit_shape* s, float* dFC, const float* In, const float* dLdO, const float* FT,
                              const float* FY, const float* FX) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad, R = s->Rank;
  float* SHIn = padded_copy(s, In);
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned c = 0; c < s->C; ++c)
    for (unsigned r = 0; r < R; ++r) {
      float a = dFC[c * R + r];
      for (unsigned n = 0; n < s->N; ++n)
        for (unsigned t = 0; t < s->T; ++t)
          for (unsigned h = 0; h < s->H; ++h)
            for (unsigned w = 0; w < s->W; ++w)
              for (unsigned y = 0; y < s->Y; ++y)
                for (unsigned x = 0; x < s->X; ++x)
                  a += DLDO(n, t, h, w) * SHIN(n, c, h + y, w + x) * FT[t * R + r] * FY[y * R + r] * FX[x * R + r];
      dFC[c * R + r] = a;
    }
  free(SHIn);
}

void cp4lit_backward_filter_y(const cp4lit_shape* s, float* dFY, const float* In, const float* dLdO, const float* FT,
                              const float* FC, const float* FX) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad, R = s->Rank;
  float* SHIn = padded_copy(s, In);
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned y = 0; y < s->Y; ++y)
    for (unsigned r = 0; r < R; ++r) {
      float a = dFY[y * R + r];
      for (unsigned n = 0; n < s->N; ++n)
        for (unsigned t = 0; t < s->T; ++t)
          for (unsigned c = 0; c < s->C; ++c)
            for (unsigned h = 0; h < s->H; ++h)
              for (unsigned w = 0; w < s->W; ++w)
                for (unsigned x = 0; x < s->X; ++x)
                  a += DLDO(n, t, h, w) * SHIN(n, c, h + y, w + x) * FT[t * R + r] * FC[c * R + r] * FX[x * R + r];
      dFY[y * R + r] = a;
    }
  free(SHIn);
}

void cp4lit_backward_filter_x(const cp4lit_shape* s, float* dFX, const float* In, const float* dLdO, const float* FT,
                              const float* FC, const float* FY) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad, R = s->Rank;
  float* SHIn = padded_copy(s, In);
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned x = 0; x < s->X; ++x)
    for (unsigned r = 0; r < R; ++r) {
      float a = dFX[x * R + r];
      for (unsigned n = 0; n < s->N; ++n)
        for (unsigned t = 0; t < s->T; ++t)
          for (unsigned c = 0; c < s->C; ++c)
            for (unsigned h = 0; h < s->H; ++h)
              for (unsigned w = 0; w < s->W; ++w)
                for (unsigned y = 0; y < s->Y; ++y)
                  a += DLDO(n, t, h, w) * SHIN(n, c, h + y, w + x) * FT[t * R + r] * FC[c * R + r] * FY[y * R + r];
      dFX[x * R + r] = a;
    }
  free(SHIn);
}

void cp4lit_backward_filter_full(const cp4lit_shape* s, float* FF, const float* In, const float* dLdO) {
  const unsigned sH = s->H + 2 * s->pad, sW = s->W + 2 * s->pad;
  float* SHIn = padded_copy(s, In);
#pragma omp parallel for collapse(2) schedule(static)
  for (unsigned t = 0; t < s->T; ++t)
    for (unsigned c = 0; c < s->C; ++c)
      for (unsigned y = 0; y < s->Y; ++y)
        for (unsigned x = 0; x < s->X; ++x) {
          float a = FF[((t * s->C + c) * s->Y + y) * s->X + x];
          for (unsigned n = 0; n < s->N; ++n)
            for (unsigned h = 0; h < s->H; ++h)
              for (unsigned w = 0; w < s->W; ++w) a += DLDO(n, t, h, w) * SHIN(n, c, h + y, w + x);
          FF[((t * s->C + c) * s->Y + y) * s->X + x] = a;
        }
  free(SHIn);
}
