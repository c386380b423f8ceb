"""The tolerances of the tests, fixed once.

Errors are the largest absolute difference of logits divided by the largest
absolute reference logit of the compared block.
- 32-bit engine against the 64-bit plain implementation: 1e-4.
- bfloat16 engine against the 64-bit plain implementation reading the same
  (bfloat16-stored) weights: 3e-2 (bfloat16 keeps 8 bits; a layer rounds about
  ten times).
- Two ways of cutting the same work in the engine itself: 2e-5 in 32-bit (kernels
  of prefill and decode add in different orders), 2e-2 in bfloat16.
"""
FP32_VS_PLAIN = 1e-4
BF16_VS_PLAIN = 3e-2
FP32_SPLITS = 2e-5
BF16_SPLITS = 2e-2

VS_PLAIN = {"float32": FP32_VS_PLAIN, "bfloat16": BF16_VS_PLAIN}
SPLITS = {"float32": FP32_SPLITS, "bfloat16": BF16_SPLITS}


def rel_err(got, ref) -> float:
    ref = ref.double()
    return float((got.double().cpu() - ref.cpu()).abs().max() / ref.abs().max().clamp_min(1e-30))
