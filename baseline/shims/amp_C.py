"""Stand-in for apex's amp_C extension: the two multi-tensor functions the reference runtime calls
(optimizer/clip_grads.py:90-118, optimizer/optimizer.py:57-60, utils.py:162-167), on torch._foreach_* kernels."""
import torch


def multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor=False):
    """Returns (global L2 norm as a 1-element fp32 tensor, per-tensor norms or None)."""
    tensors = tensor_lists[0]
    if not tensors:
        dev = noop_flag.device
        return torch.zeros(1, dtype=torch.float32, device=dev), None
    norms = torch._foreach_norm(tensors, 2.0)
    stacked = torch.stack([n.float() for n in norms])
    total = torch.linalg.vector_norm(stacked, 2.0).reshape(1)
    return total, (stacked if per_tensor else None)


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    """dst[i] = src[i] * scale (with a dtype cast when the lists differ); sets noop_flag when a value is not finite."""
    src, dst = tensor_lists
    if not src:
        return
    if src is dst or all(a is b for a, b in zip(src, dst)):
        torch._foreach_mul_(dst, scale)
    else:
        torch._foreach_copy_(dst, src)
        if scale != 1.0:
            torch._foreach_mul_(dst, scale)
