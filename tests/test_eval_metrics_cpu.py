"""``MerakTrainer.evaluation`` with ``return_logits`` + ``compute_metrics``: the reported accuracy equals the
one computed directly from the model's logits on the evaluation set, and ``eval_batch`` hands back
``(loss, logits, labels)`` per micro-batch (reference behaviour: Merak/core/merak_engine.py:1271-1360)."""
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

import merak_b200 as Merak


class _Set(torch.utils.data.Dataset):
    def __init__(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(n, 16, generator=g)
        self.y = (self.x[:, 0] > 0).long()            # learnable, so that the accuracy is not trivially 0 or 1

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return {"x": self.x[i], "labels": self.y[i]}


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b = nn.Linear(16, 32), nn.Linear(32, 2)

    def forward(self, x):
        return self.b(torch.tanh(self.a(x)))


def test_evaluation_accuracy_matches_direct_computation(tmp_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29000 + os.getpid() % 1000), RANK="0", WORLD_SIZE="1",
                      LOCAL_RANK="0", MERAK_QUIET="1")
    Merak.init(1, 1, 1, backend="gloo")
    try:
        torch.manual_seed(0)
        model = _Net()
        args = Merak.MerakArguments(output_dir=str(tmp_path), per_device_train_batch_size=8, per_device_eval_batch_size=8,
                                    gradient_accumulation_steps=2, max_steps=20, learning_rate=5e-2, logging_steps=0,
                                    no_cuda=True, report_to="none", seed=1, return_logits=True, input_names=["x"],
                                    lr_scheduler_type="constant", weight_decay=0.0)
        evald = _Set(64, 7)
        seen = []

        def compute_metrics(p):
            seen.append((p.predictions.shape, p.label_ids.shape))
            return {"accuracy": (p.predictions.argmax(-1) == p.label_ids).float().mean().item()}

        trainer = Merak.MerakTrainer(model, args, train_dataset=_Set(256, 3), eval_dataset=evald,
                                     compute_metrics=compute_metrics,
                                     loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
        trainer.train()
        loss = trainer.evaluation()
        # every evaluation step hands over its micro-batches' logits and labels: 2 x 8 samples per step, 4 steps
        assert seen and all(ps == (16, 2) and ls == (16,) for ps, ls in seen) and len(seen) == 4, seen
        engine = trainer.engine
        engine.module.eval()
        with torch.no_grad():
            logits = torch.cat([engine.module((), {"x": evald.x[i:i + 8]}) for i in range(0, 64, 8)])
        direct_acc = (logits.argmax(-1) == evald.y).float().mean().item()
        direct_loss = F.cross_entropy(logits, evald.y).item()
        assert abs(trainer.eval_metrics["accuracy"] - direct_acc) < 1e-6, (trainer.eval_metrics, direct_acc)
        assert abs(loss - direct_loss) < 1e-4, (loss, direct_loss)
        assert direct_acc > 0.7, direct_acc           # the task was learned, so the comparison is not vacuous
        # the engine call itself
        it = iter([{"x": evald.x[:8], "labels": evald.y[:8]}, {"x": evald.x[8:16], "labels": evald.y[8:16]}])
        l, lg, lb = engine.eval_batch(it)
        assert len(lg) == 2 and len(lb) == 2 and torch.equal(lb[1], evald.y[8:16])
        assert torch.allclose(torch.cat(lg), logits[:16], atol=1e-6) and float(l) > 0
    finally:
        Merak.initialize.destroy()


def test_eval_strategy_arguments_and_step_evaluation(tmp_path):
    """``--evaluation_strategy`` (the spelling of the reference's READMEs) / ``--eval_strategy``: ``steps``
    evaluates every ``eval_steps`` optimizer steps, ``epoch`` after every pass over the data; ``do_eval`` alone
    means ``epoch``; ``--input_name`` abbreviates ``--input_names`` as in the reference's command lines."""
    from merak_b200.args import MerakArguments, parse_args
    a = parse_args(["--evaluation_strategy=epoch", "--no_cuda", "true", "--input_name", "x", "y"])
    assert (a.eval_strategy, a.do_eval, a.input_names) == ("epoch", True, ["x", "y"])
    b = MerakArguments(no_cuda=True, eval_strategy="steps", logging_steps=7)
    assert (b.eval_steps, b.do_eval) == (7, True)
    assert MerakArguments(no_cuda=True, do_eval=True).eval_strategy == "epoch"
    assert MerakArguments(no_cuda=True).do_eval is False

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29000 + (os.getpid() + 5) % 1000), RANK="0",
                      WORLD_SIZE="1", LOCAL_RANK="0", MERAK_QUIET="1")
    Merak.init(1, 1, 1, backend="gloo")
    try:
        args = Merak.MerakArguments(output_dir=str(tmp_path), per_device_train_batch_size=8, per_device_eval_batch_size=8,
                                    gradient_accumulation_steps=1, max_steps=10, logging_steps=0, no_cuda=True,
                                    report_to="none", input_names=["x"], eval_strategy="steps", eval_steps=5)
        trainer = Merak.MerakTrainer(_Net(), args, train_dataset=_Set(256, 3), eval_dataset=_Set(16, 7),
                                     loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
        at_steps = []
        plain = trainer.evaluation
        trainer.evaluation = lambda *a, **k: (at_steps.append(trainer.params.global_steps), plain(*a, **k))[1]
        trainer.train()
        assert at_steps == [5, 10], at_steps
        # without the ``steps`` strategy ``eval_steps`` is the length of one evaluation, as in the reference
        args.eval_strategy, args.eval_steps = "no", 1
        calls, eval_batch = [], trainer.engine.eval_batch
        trainer.engine.eval_batch = lambda *a, **k: (calls.append(1), eval_batch(*a, **k))[1]
        plain()
        assert len(calls) == 1, calls
    finally:
        Merak.initialize.destroy()
