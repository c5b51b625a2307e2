"""Greedy decoding through the training pipeline (forward-only DualPipeV), as a check of converted weights.

    python examples/inference/greedy_decode.py --model examples/pretrain_lm/qwen3-30b-a3b/config.json \
        --checkpoint workspace/checkpoints/qwen3-30b-a3b/torch-dcp/step-00000000 --prompt-ids 9707,11,1879 --new-tokens 16
    torchrun --nproc-per-node 8 examples/inference/greedy_decode.py ... --pp 2 --ep 4

The sequence length is static (``--seq``): the prompt is right-padded, every step runs the whole padded sequence with
``DualPipeV.step`` under ``no_grad`` and ``return_outputs=True`` and reads the logits at the last real position — no KV
cache, which is fine for a coherence check of a few dozen tokens. Without ``--checkpoint`` the seeded random
initialisation is used (the output is then meaningless but the path is exercised). ``--num-hidden-layers`` truncates
the model for a quick run. The role of the reference's inference template
(.agents/skills/add-new-model/templates/inference_test.py).
"""

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from pithtrain_b200.contexts import distributed, training  # noqa: E402
from pithtrain_b200.modules.distributed import setup_distributed  # noqa: E402
from pithtrain_b200.modules.logging import setup_logging  # noqa: E402
from pithtrain_b200.modules.training import make_adamw_optimizer, make_constant_scheduler, setup_training  # noqa: E402
from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--checkpoint", default=None, help="DCP directory (step-XXXXXXXX) with canonical model keys")
    ap.add_argument("--prompt-ids", default="1,2,3,4")
    ap.add_argument("--new-tokens", type=int, default=8)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--num-hidden-layers", type=int, default=0)
    a = ap.parse_args()

    cfg = PretrainLMCfg()
    cfg.distributed.pipeline_parallel_size, cfg.distributed.expert_parallel_size = a.pp, a.ep
    t = cfg.training
    t.model, t.dataset = Path(a.model), None
    t.sequence_length, t.micro_batch_size = a.seq, 1
    t.global_batch_size = 2 * a.pp * a.ep  # the pipeline wants at least 2·pp micro-batches; all carry the same prompt
    t.optimizer, t.scheduler, t.lr, t.max_steps = make_adamw_optimizer, make_constant_scheduler, 0.0, 1
    if a.num_hidden_layers:
        t.num_hidden_layers_override = a.num_hidden_layers
    setup_logging(cfg)
    setup_distributed(cfg)
    setup_training(cfg)
    if a.checkpoint:
        from pithtrain_b200.modules.checkpoint import load_into

        load_into(Path(a.checkpoint), training.model)
    model = training.model
    model.eval()
    dev = distributed.device
    ids = [int(x) for x in a.prompt_ids.split(",") if x.strip()]
    assert 0 < len(ids) < a.seq
    chunks = 2 * a.pp
    for _ in range(a.new_tokens):
        if len(ids) >= a.seq:
            break
        row = torch.zeros(a.seq, dtype=torch.long)
        row[: len(ids)] = torch.tensor(ids)
        batch = row.unsqueeze(0).repeat(chunks, 1).to(dev)
        with torch.no_grad():
            _, logits = model.step(batch if distributed.pp_rank == 0 else None, num_chunks=chunks, return_outputs=True)
        nxt = torch.zeros(1, dtype=torch.long, device=dev)
        if distributed.pp_rank == 0:
            nxt[0] = logits[0, len(ids) - 1].float().argmax()
        if distributed.world_size > 1:
            torch.distributed.broadcast(nxt, src=0)
        ids.append(int(nxt))
    if distributed.rank == 0:
        print("token ids:", ",".join(str(i) for i in ids))


if __name__ == "__main__":
    main()
