"""DeepSeek-V2-Lite-shape mixture-of-experts LM with expert parallelism (``EP`` ranks of every
data-parallel group share the routed experts).  Not among the reference's examples: it has no MoE.

    EP=8 torchrun --nproc_per_node=8 --master-addr 127.0.0.1 examples/models/moe/run_moe.py --bf16 true ...
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from _common import degrees, parse

import merak_b200 as Merak
from merak_b200.models.moe import DeepseekV2ForCausalLM, deepseek_v2_config
from merak_b200.utils.datasets import SyntheticTokenDataset


def main():
    args, own = parse({"model_size": "deepseek-v2-lite", "seq_length": 4096, "dataset_size": 1024, "num_layers_override": 0})
    Merak.init(**degrees())
    over = {"num_hidden_layers": own.num_layers_override} if own.num_layers_override else {}
    config = deepseek_v2_config(own.model_size, **over)
    model = DeepseekV2ForCausalLM(config)
    train = SyntheticTokenDataset(config.vocab_size, min(own.seq_length, config.max_position_embeddings),
                                  own.dataset_size, task="causal", seed=args.seed)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train)
    trainer.train()


if __name__ == "__main__":
    main()
