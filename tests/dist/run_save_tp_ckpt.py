"""Worker (torchrun, gloo, CPU): a tensor-parallel model writes its per-rank checkpoint and strategy files and the
loss of one fixed batch, for the resharding test to load under another layout."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.checkpoint.io import save_checkpoint  # noqa: E402
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.layers.gpt_model import GPTModel  # noqa: E402
from mindformers_b200.parallel.transformer_config import TransformerConfig  # noqa: E402

CFG = dict(num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=256,
           vocab_size=512, seq_length=64, max_position_embeddings=64, params_dtype="float32", compute_dtype="float32",
           layernorm_epsilon=1e-5, pad_token_id=-1)


def batch():
    ids = torch.randint(0, 512, (2, 33), generator=torch.Generator().manual_seed(99))
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def main():
    out = sys.argv[1]
    dist.init_process_group("gloo")
    world = dist.get_world_size()
    ps.initialize_model_parallel(tensor_model_parallel_size=world)
    torch.manual_seed(31)
    cfg = TransformerConfig(tensor_model_parallel_size=world, **CFG)
    cfg.device = "cpu"
    model = GPTModel(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():                      # move away from the initial values, identically on all ranks
            p.mul_(1.5)
        inp, lab = batch()
        loss = float(model(inp, labels=lab))
    save_checkpoint(model, os.path.join(out, "checkpoint"), epoch=1, step=7, extra={"global_batch_size": 16})
    if dist.get_rank() == 0:
        json.dump({"loss": loss}, open(os.path.join(out, "loss.json"), "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
