// The gated unit between the two products of a gated feed-forward, from the float32 sums g (gate) and u (up) and a
// weight w of the row (1 where there is none).  Two kinds:
//   MLXB_GU_SILU     silu(w g) * (w u): the unit of the input scaled by w (the products are linear in it);
//   MLXB_GU_BOUNDED  with g' = min(g, limit) and u' = clamp(u, -limit, limit): w * g' * sigmoid(1.702 g') * (u' + 1),
//                    the unit's output scaled by w.
#pragma once

enum { MLXB_GU_SILU = 0, MLXB_GU_BOUNDED = 1 };

__device__ __forceinline__ float mlxb_gated_unit(int kind, float g, float u, float w, float limit) {
  if (kind == MLXB_GU_BOUNDED) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return w * (g / (1.f + expf(-1.702f * g))) * (u + 1.f);
  }
  const float a = w * g;
  return (a / (1.f + expf(-a))) * (w * u);
}
