// The shaping of attention scores on their way to the softmax, shared by the attention kernels over [key | value] rows.
#pragma once

// What a mixer may do to a score between the scaled dot product and the softmax, in this order: a factor
// per query head, a soft cap (cap * tanh(s / cap)), and a bias that grows with the distance between query
// and key (s - slope_h * (i - j)).  Null pointers and a cap of 0 leave the score as it is.  out_scale
// multiplies the attention's result (the weight of this mixer where two run side by side).
struct ScoreShape {
  const float* head_scale;   // [heads] or null
  const float* slopes;       // [heads] or null
  float softcap;             // 0: none
  float out_scale;           // 1: none
};

__device__ __forceinline__ float shape_score(float s, const ScoreShape& sh, int head, int dist) {
  if (sh.head_scale != nullptr) s *= sh.head_scale[head];
  if (sh.softcap > 0.f) s = sh.softcap * tanhf(s / sh.softcap);
  if (sh.slopes != nullptr) s = fmaf(-sh.slopes[head], (float)dist, s);
  return s;
}
