"""Stand-in for the parts of NVIDIA apex that the reference runtime imports (runtime/megatron/optimizer/__init__.py:16-17,
optimizer/clip_grads.py:21-22, optimizer/optimizer.py:23-24, utils.py:31-32).  apex is not in this image; the stand-ins
run on torch's own fused multi-tensor kernels, so the reference's optimizer step stays a handful of launches as with apex."""
