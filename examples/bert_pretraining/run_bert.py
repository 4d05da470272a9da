"""BERT-large masked-LM pre-training with a user optimizer (LAMB), a user learning-rate schedule and a
user loss, all supplied through trainer hooks (the reference's examples/bert_pretraining/run_bert.py:
61-117: init(2,1,2)).  Data are generated token ids with the 80/10/10 masking rule."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import degrees, parse

import merak_b200 as Merak
from lamb import Lamb
from merak_b200.models.bert import BertForMaskedLM, bert_config
from merak_b200.ops.cross_entropy import softmax_cross_entropy
from merak_b200.utils.datasets import SyntheticTokenDataset
from schedulers import PolyWarmUpScheduler


class BertPretrainingTrainer(Merak.MerakTrainer):
    def create_optimizer(self, params):
        return Lamb(params, lr=self.args.learning_rate, weight_decay=self.args.weight_decay,
                    max_grad_norm=self.args.max_grad_norm)

    def create_lr_scheduler(self, optimizer):
        return PolyWarmUpScheduler(optimizer, warmup=0.1, total_steps=max(1, self.params.max_steps or 1000))

    def get_loss_fn(self):
        def mlm_loss(outputs, labels):
            logits = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
            return softmax_cross_entropy(logits, labels)        # labels are -100 off the masked positions
        return mlm_loss


def main():
    args, own = parse({"model_size": "bert-large", "seq_length": 512, "dataset_size": 8192})
    Merak.init(**degrees())
    config = bert_config(own.model_size)
    model = BertForMaskedLM(config)
    train = SyntheticTokenDataset(config.vocab_size, min(own.seq_length, config.max_position_embeddings),
                                  own.dataset_size, task="mlm", seed=args.seed)
    BertPretrainingTrainer(model, args, train_dataset=train).train()


if __name__ == "__main__":
    main()
