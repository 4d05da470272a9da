"""BERT masked-language-model training on generated data with tensor parallelism from the built-in
feature table (the reference's examples/models/bert: init(2,2,1))."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from _common import degrees, parse

import merak_b200 as Merak
from merak_b200.models.bert import BertForMaskedLM, bert_config
from merak_b200.utils.datasets import SyntheticTokenDataset


def main():
    args, own = parse({"model_size": "bert-large", "seq_length": 512, "dataset_size": 8192})
    Merak.init(**degrees())
    config = bert_config(own.model_size)
    model = BertForMaskedLM(config)
    train = SyntheticTokenDataset(config.vocab_size, min(own.seq_length, config.max_position_embeddings),
                                  own.dataset_size, task="mlm", seed=args.seed)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train)
    trainer.train()


if __name__ == "__main__":
    main()
