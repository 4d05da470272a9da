"""LoRA fine-tuning: low-rank adapters are injected into the attention projections, only they are
trained and saved (``lora_`` checkpoint files plus ``lora_config.json``), and a later run resumes
from them (the reference's examples/lora/run_vit.py:89-316 and examples/deepseek-r1/finetune.py:
125-227 do this for ViT and for Llama/Qwen distillations; the model here is the framework's Llama).

    python examples/lora/run_lora.py --lora_config examples/lora/lora_config.json --output_dir ./out ...
    # base weights: --resume_from_checkpoint <Hugging Face directory or a framework checkpoint>
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

import merak_b200 as Merak
from merak_b200.models.llama import LlamaForCausalLM, llama_config
from merak_b200.utils.datasets import SyntheticTokenDataset


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    args, own = parse({"model_size": "llama-7b", "seq_length": 1024, "dataset_size": 2048,
                       "lora_config": os.path.join(here, "lora_config.json")})
    Merak.init(**degrees())
    config = llama_config(own.model_size)
    model = LlamaForCausalLM(config)
    train = SyntheticTokenDataset(config.vocab_size, min(args.seq_length or own.seq_length, config.max_position_embeddings),
                                  own.dataset_size, task="causal", seed=args.seed)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train)
    trainer.train()
    trainable = sum(p.numel() for p in trainer.engine.module.parameters() if p.requires_grad)
    total = sum(p.numel() for p in trainer.engine.module.parameters())
    if Merak.mpu.get_global_rank() == 0:
        print("trainable parameters on this stage: %d of %d" % (trainable, total))


if __name__ == "__main__":
    main()
