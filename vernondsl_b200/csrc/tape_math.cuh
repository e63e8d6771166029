// Elementwise primitives shared by the compiled map kernels and by the kernels that the tape
// compiler generates at run time: this file is included by k_map.cu and, as text, handed to NVRTC
// in front of every generated kernel, so that both paths round identically.  It must stay free of
// #include lines and of anything that is not available to a run-time compiled translation unit.
#ifndef VRHI_TAPE_MATH_CUH
#define VRHI_TAPE_MATH_CUH

// exp(x) to well under one ulp in the normal range: n = round(x*log2e), r = x - n*ln2 with a
// two-constant split (both steps exact or fused), exp(r) = 1 + (r + r*r*q(r)) with the Taylor
// polynomial through r^7 (|r| <= 0.3466, next term < 2^-27), scaled by 2^n in two exact factors.
__device__ __forceinline__ float exp_sub_ulp(float x) {
  x = fminf(fmaxf(x, -104.0f), 88.72f);
  const float t = fmaf(x, 1.442695041f, 12582912.0f);
  const float n = t - 12582912.0f;
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-06f, r);
  float q = 1.98412698e-4f;
  q = fmaf(q, r, 1.38888889e-3f);
  q = fmaf(q, r, 8.33333333e-3f);
  q = fmaf(q, r, 4.16666667e-2f);
  q = fmaf(q, r, 1.66666667e-1f);
  q = fmaf(q, r, 0.5f);
  const float p = fmaf(r * r, q, r);
  const float res = 1.0f + p;
  const int ni = (int)n, h = ni / 2;
  return res * __int_as_float((h + 127) << 23) * __int_as_float((ni - h + 127) << 23);
}

// 1 / (1 + exp(-x)): the rounding of 1 + E is recovered (two-sum) and folded into one Newton
// step on the reciprocal, so that the result carries little more than the error of E itself.
__device__ __forceinline__ float sigmoid_accurate(float x) {
  const float e = exp_sub_ulp(-x);
  const float d = 1.0f + e;
  const float dl = (e > 1.0f) ? (e - d) + 1.0f : (1.0f - d) + e;
  const float r = 1.0f / d;
  const float err = fmaf(-d, r, 1.0f);
  return fmaf(r, err - dl * r, r);
}

#endif  // VRHI_TAPE_MATH_CUH
