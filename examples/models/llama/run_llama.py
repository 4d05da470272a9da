"""Llama-shape causal LM with a hand-written tensor-parallel layer table and the attention block kept
as a tracing leaf (the reference's examples/models/llama/run_llama.py:46-93: init(4,2,1))."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from _common import degrees, parse

import merak_b200 as Merak
from merak_b200.models.llama import LlamaAttention, LlamaForCausalLM, llama_config
from merak_b200.parallel.tp_transform import set_tp_layer_lists
from merak_b200.utils.datasets import DynamicGenDataset


def main():
    args, own = parse({"model_size": "llama-7b", "seq_length": 2048, "dataset_size": 2048})
    Merak.init(**degrees())
    config = llama_config(own.model_size)
    model = LlamaForCausalLM(config)
    # which Linear layers become column / row parallel, and which integer attributes shrink with tp
    set_tp_layer_lists(col_para_list=["qkv_proj", "gate_up_proj"], row_para_list=["o_proj", "down_proj"],
                       tp_attr_list=["num_heads", "num_key_value_heads"])
    train = DynamicGenDataset(config, mode="text_only", dataset_size=own.dataset_size,
                              seq_length=min(own.seq_length, config.max_position_embeddings))
    trainer = Merak.MerakTrainer(model, args, train_dataset=train, leaf_modules=(LlamaAttention,))
    trainer.train()


if __name__ == "__main__":
    main()
