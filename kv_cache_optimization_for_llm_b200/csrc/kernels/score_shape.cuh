// The shaping of attention scores on their way to the softmax, shared by the attention kernels over [key | value] rows.
#pragma once

// What a mixer may do to a score between the scaled dot product and the softmax, in this order: a factor
// per query head, a soft cap (cap * tanh(s / cap)), and a bias that grows with the distance between query
// and key (s - slope_h * (i - j)).  Null pointers and a cap of 0 leave the score as it is.  out_scale
// multiplies the attention's result (the weight of this mixer where two run side by side).
// Further, for the kernels that take them (those of window_attention.cu): `sinks`, a learned score per head that
// joins the softmax's denominator once and has no value (exp(sink_h) beside the keys' exp(s)); `chunk`, a mask by
// blocks of positions counted from the sequence's start (query i sees key j <= i only when i / chunk == j / chunk);
// and `gate`, rows in the activations' type by whose sigmoid the result is multiplied element by element
// (gate[t * gate_ld + head * Dv + i]).  Members left out of an initialiser are null or 0: absent.
struct ScoreShape {
  const float* head_scale;   // [heads] or null
  const float* slopes;       // [heads] or null
  float softcap;             // 0: none
  float out_scale;           // 1: none
  const float* sinks;        // [heads] or null
  int chunk;                 // 0: none
  const void* gate;          // [T, >= heads * Dv] or null
  int gate_ld;
};

// The first key that position `pos` sees: the window's and the block's lower ends, whichever is later.
__device__ __forceinline__ int first_seen_key(int pos, int window, int chunk) {
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (chunk > 0) lo = max(lo, pos - pos % chunk);
  return lo;
}

__device__ __forceinline__ float shape_score(float s, const ScoreShape& sh, int head, int dist) {
  if (sh.head_scale != nullptr) s *= sh.head_scale[head];
  if (sh.softcap > 0.f) s = sh.softcap * tanhf(s / sh.softcap);
  if (sh.slopes != nullptr) s = fmaf(-sh.slopes[head], (float)dist, s);
  return s;
}
