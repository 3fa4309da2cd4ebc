"""Peak-memory probe for tensor parallelism (run with torchrun on 2 GPUs):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        scripts/measure_tp_memory.py --tokens 8192

Builds a random Qwen3-style model, shards it over the two ranks and reports the peak allocated
memory of one forward+backward (counterpart of the reference's scripts/measure_tp_memory.py)."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2560)
    args = ap.parse_args()
    dist.init_process_group("nccl")
    rank = dist.get_rank()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    from lset_b200.dist.tp import apply_tp
    from lset_b200.models import Qwen3Config, Qwen3Decoder
    from lset_b200.models.parallel_plan import decoder_tp_plan

    cfg = Qwen3Config(vocab_size=32000, hidden_size=args.hidden, intermediate_size=4 * args.hidden - args.hidden // 4 * 1,
                      num_hidden_layers=args.layers, num_attention_heads=args.hidden // 128 * 1,
                      num_key_value_heads=8, head_dim=128)
    for tp in (False, True):
        torch.manual_seed(0)
        model = Qwen3Decoder(cfg, fused_projections=True).to("cuda", torch.bfloat16)
        if tp:
            apply_tp(model, dist.group.WORLD, decoder_tp_plan(cfg, fused_projections=True))
        torch.cuda.reset_peak_memory_stats()
        ids = torch.randint(0, 32000, (args.tokens,), device="cuda")
        cu = torch.tensor([0, args.tokens], dtype=torch.int32, device="cuda")
        out = model(ids, cu_seqlens=cu, max_seqlen=args.tokens)["hidden_states"]
        out.float().pow(2).mean().backward()
        torch.cuda.synchronize()
        if rank == 0:
            print(f"tp={'2' if tp else '1'} peak allocated: {torch.cuda.max_memory_allocated() / 2**30:.2f} GiB")
        del model, out
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
