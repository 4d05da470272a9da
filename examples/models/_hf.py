"""Shared body of the Hugging Face example scripts: build a ``transformers`` model from a config
(random weights; a tiny configuration with ``--tiny 1`` so the script also runs on a laptop CPU),
feed it generated data of the right modality (``DynamicGenDataset``) and train it through the
trainer.  The model is traced with ``torch.export`` and folded back into a module graph
(``merak_b200/fx/export_trace.py``), then sharded, partitioned and tensor-parallelised like the
framework's own models.  One file per model family in the sub-directories, as in the reference's
``examples/models/*``."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse  # noqa: E402

import merak_b200 as Merak  # noqa: E402
from merak_b200.utils.datasets import DynamicGenDataset  # noqa: E402

TINY = dict(
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, intermediate_size=128, max_position_embeddings=64,
    vocab_size=512, n_layer=2, n_embd=64, n_head=4, n_positions=64, n_inner=128, num_layers=2, num_decoder_layers=2,
    d_model=64, num_heads=4, d_kv=16, d_ff=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
    decoder_attention_heads=4, encoder_ffn_dim=128, decoder_ffn_dim=128, ffn_dim=128, embedding_size=32,
    num_key_value_heads=2, image_size=32, patch_size=8, num_labels=10, hidden_sizes=[16, 32], depths=[1, 1],
    rotary_dim=8, dim=64, n_heads=4, n_layers=2, hidden_dim=128, word_embed_proj_dim=64, true_hidden_size=64,
    intra_bottleneck_size=32, num_feedforward_networks=1, max_2d_position_embeddings=128,
)


class _Mapped:
    """A dataset whose samples pass through ``fn`` (sample dict -> sample dict)."""

    def __init__(self, base, fn):
        self.base, self.fn = base, fn

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.fn(self.base[i])


def run(config_cls, model_cls, mode="text_only", tp_lists=None, defaults=None, config_overrides=None,
        tiny_overrides=None, loss_fn=None, sample_fn=None, num_layers=None):
    """``tp_lists``: (column-parallel names, row-parallel names) for models without a built-in feature
    dict, the counterpart of the reference scripts' ``set_tp_layer_lists`` calls
    (examples/models/llama/run_llama.py:60-68).  ``tiny_overrides``: configuration fields of the ``--tiny 1``
    shape that are specific to the family (per-stage lists, token ids).  ``loss_fn``: ``model -> loss(outputs,
    labels)`` for heads whose loss is not a token cross entropy (CTC), the counterpart of the reference scripts'
    ``get_loss_fn`` overrides (examples/models/wav2vec2/run_wav2vec2.py:72-119).  ``sample_fn``: applied to
    every generated sample (feature layout fixes).  ``num_layers``: the depth the partitioner should assume when
    the configuration does not state it as one number."""
    import inspect
    extra = {"tiny": 0, "seq_length": 128, "dataset_size": 512}
    extra.update(defaults or {})
    args, own = parse(extra)
    if num_layers is not None and getattr(args, "num_layers", None) is None:
        args.num_layers = num_layers       # for configurations whose depth is not one integer field
    Merak.init(**degrees())
    kw = {}
    if own.tiny:
        accepted = set(inspect.signature(config_cls.__init__).parameters)
        probe = config_cls()
        kw.update({k: v for k, v in TINY.items() if k in accepted or hasattr(probe, k)})
        kw.update(tiny_overrides or {})          # family-specific shapes (per-stage lists and the like)
        kw = {k: v for k, v in kw.items() if v is not None}      # None drops a generic field (aliases of list fields)
        own.seq_length = min(own.seq_length, 32)
    kw.update(config_overrides or {})
    config = config_cls(**kw)
    for name in ("hidden_dropout_prob", "attention_probs_dropout_prob", "dropout", "attention_dropout",
                 "activation_dropout", "resid_pdrop", "embd_pdrop", "attn_pdrop", "dropout_rate", "classifier_dropout"):
        if own.tiny and hasattr(config, name) and getattr(config, name) is not None:
            setattr(config, name, 0.0)
    model = model_cls(config)
    if tp_lists is not None:
        from merak_b200.parallel.tp_transform import set_tp_layer_lists
        set_tp_layer_lists(col_para_list=tp_lists[0], row_para_list=tp_lists[1])
    train = DynamicGenDataset(config, mode=mode, dataset_size=own.dataset_size, seq_length=own.seq_length)
    if sample_fn is not None:       # reshape generated samples into what this family's forward expects
        train = _Mapped(train, sample_fn)
    trainer = Merak.MerakTrainer(model, args, train_dataset=train,
                                 loss_fn=loss_fn(model) if loss_fn is not None else None)
    trainer.train()
    return trainer
