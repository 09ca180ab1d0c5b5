"""Worker (torchrun, gloo, CPU): the dropless all-to-all MoE gives the same result with experts split over two ranks
as with all experts on one rank, forward and input gradient."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.modules import MoEConfig, MoEV3  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    cfg = MoEConfig(expert_num=4, num_experts_chosen=2, moe_intermediate_size=24)
    torch.manual_seed(7)
    sharded = MoEV3(16, 24, cfg, group=dist.group.WORLD)
    torch.manual_seed(7)
    full = MoEV3(16, 24, cfg, group=None)
    assert sharded.w1.shape[0] == 2 and torch.equal(sharded.w1, full.w1[rank * 2:rank * 2 + 2])
    g = torch.Generator().manual_seed(100 + rank)                     # every rank has its own tokens
    x = torch.randn(3 + 2 * rank, 5, 16, generator=g, requires_grad=True)
    x_ref = x.detach().clone().requires_grad_(True)
    y, aux = sharded(x)
    y_ref, aux_ref = full(x_ref)
    assert torch.allclose(y, y_ref, atol=1e-5) and torch.allclose(aux, aux_ref)
    y.square().sum().backward()
    y_ref.square().sum().backward()
    assert torch.allclose(x.grad, x_ref.grad, atol=1e-5)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
