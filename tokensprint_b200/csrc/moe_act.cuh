// What the expert kernels of both kinds (CUDA cores, tensor cores) share: the gated activations
// and the ways a router turns chosen logits into weights.
#pragma once

#define MOE_ACT_CAPPED_GLU 0  // a = min(g, limit), b = clamp(u, -limit, limit): a * sigmoid(alpha a) * (b + 1)
#define MOE_ACT_SWIGLU 1      // g * sigmoid(g) * u  (limit and alpha unused)
#define MOE_ACT_GELU 2        // experts without a gate matrix: gelu(u) in its exact (erf) form; g is not read

__device__ __forceinline__ float moe_gated_activation(int mode, float g, float u, float limit, float alpha) {
  if (mode == MOE_ACT_SWIGLU) return g / (1.f + expf(-g)) * u;
  if (mode == MOE_ACT_GELU) return 0.5f * u * (1.f + erff(u * 0.70710678118654752f));
  const float a = fminf(g, limit);
  const float b = fminf(fmaxf(u, -limit), limit);
  return a / (1.f + expf(-alpha * a)) * (b + 1.f);
}

#define ROUTER_SCORE_SIGMOID 0        // weight = sigmoid(logit), optionally divided by the chosen ones' sum
#define ROUTER_SCORE_SOFTMAX_CHOSEN 1 // weight = softmax over the chosen logits only
#define ROUTER_SCORE_SOFTMAX_ALL 2    // score = softmax over all logits; chosen by score + correction, weight = the score itself
