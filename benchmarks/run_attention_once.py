"""Launch the flash-attention forward and backward kernels a few times on one small problem
(B=1, S=4096, 32 q heads / 8 kv heads, head dim 128): the target of `ncu -k regex:flash_attn`.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.ops import attention as A  # noqa: E402

B, S, nq, nkv, hd = 1, 4096, 32, 8, 128
packed = (torch.randn(B * S, nq + 2 * nkv, hd, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
g = torch.randn(B * S, nq * hd, device="cuda", dtype=torch.bfloat16) * 0.1
for _ in range(3):
    packed.grad = None
    A.flash_attention_packed(packed, B, S, nq, nkv, True).backward(g)
torch.cuda.synchronize()
print("done")
