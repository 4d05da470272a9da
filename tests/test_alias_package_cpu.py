"""``import Merak`` and the reference's module paths resolve to this framework: every name the
reference's package ``__init__`` files export (Merak/__init__.py, Merak/utils/__init__.py,
Merak/core/__init__.py, Merak/core/*/__init__.py, Merak/inference/__init__.py,
Merak/merak_args/__init__.py) is importable from the same path, aliased modules are the same objects
as the ``merak_b200`` ones (shared state), and unknown paths fail like any missing module."""
import importlib
import sys

import pytest

EXPORTS = {
    "Merak": ["MerakTrainer", "init", "get_grid", "get_args", "get_topo", "MerakArguments", "print_rank_0",
              "init_empty_weights"],
    "Merak.utils": ["init_empty_weights", "WorkerInitObj", "MegatronPretrainingRandomSampler", "BaseParams",
                    "RepeatingLoader"],
    "Merak.utils.datasets": ["DynamicGenDataset"],
    "Merak.utils.parameters": ["BaseParams"],
    "Merak.core": ["mpu", "PipelineEngine", "recompute", "printer", "PipelineModule"],
    "Merak.core.mpu": [
        "vocab_parallel_cross_entropy", "destroy_model_parallel", "get_data_parallel_group", "get_data_parallel_rank",
        "get_data_parallel_world_size", "get_model_parallel_group", "get_model_parallel_rank",
        "get_model_parallel_src_rank", "get_model_parallel_world_size", "get_pipe_parallel_group",
        "get_pipe_parallel_rank", "get_pipe_parallel_world_size", "get_pipeline_model_parallel_prev_rank",
        "get_pipeline_model_parallel_next_rank", "is_pipeline_first_stage", "is_pipeline_last_stage",
        "get_sequence_parallel_group", "get_sequence_parallel_rank", "get_sequence_parallel_world_size", "LayerNorm",
        "ColumnParallelLinear", "RowParallelLinear", "VocabParallelEmbedding", "ColParallelConv2d",
        "copy_to_model_parallel_region", "gather_from_model_parallel_region", "reduce_from_model_parallel_region",
        "scatter_to_model_parallel_region", "all_to_all_sequence_parallel_region",
        "split_for_sequence_parallel_region", "gather_for_sequence_parallel_region", "divide",
        "split_tensor_along_last_dim"],
    "Merak.core.printer": ["SynchronizedWallClockTimer", "ThroughputTimer", "LoggerFactory", "log_dist", "logger",
                           "see_memory_usage", "set_timer_log_rank", "AccMetric"],
    "Merak.core.recompute": ["checkpoint", "pre_checkpoint", "get_rng_tracker", "RNGManager",
                             "model_parallel_cuda_manual_seed"],
    "Merak.core.checkpoint": ["CheckpointSaver", "CheckpointLoader", "rotate_checkpoints"],
    "Merak.core.pipeline": ["InferenceSchedule", "PipeSchedule", "TrainSchedule", "MergeP2PTrainSchedule",
                            "LastNoRecomputeTrainSchedule", "FullCriticalPathTrainSchedule", "PipelineModule",
                            "LayerPartition"],
    "Merak.core.fx": ["convert_to_sequential"],
    "Merak.core.fx.tracer": ["tf_symbolic_trace", "LayerProxyTracer", "dynamo_trace"],
    "Merak.core.tensor_parallel.mp_attrs": ["set_tp_layer_lists"],
    "Merak.core.zero": ["configure_zero_optimizer"],
    "Merak.core.amp": ["MixedPrecisionConfig"],
    "Merak.core.finetuning.lora": ["LoraConfig", "mark_only_lora_as_trainable", "_find_and_replace"],
    "Merak.core.sequence_parallel": ["replace_to_sp_module", "get_leaf_modules_for_sp"],
    "Merak.inference": ["text_generation_pipeline"],
    "Merak.merak_args": ["MerakArguments", "get_args", "mergeargs", "manual_set_args"],
    "Merak.merak_trainer": ["MerakTrainer"],
    "Merak.initialize": ["init", "get_grid", "get_topo", "print_rank_0"],
    "Merak.core.merak_engine": ["PipelineEngine"],
}


@pytest.mark.parametrize("path", sorted(EXPORTS))
def test_reference_exports_resolve(path):
    mod = importlib.import_module(path)
    missing = [n for n in EXPORTS[path] if not hasattr(mod, n)]
    assert not missing, (path, missing)


def test_aliases_share_objects_and_state():
    import Merak
    import merak_b200
    from Merak.core import mpu
    from merak_b200.parallel import mpu as real_mpu
    assert mpu.get_data_parallel_rank is real_mpu.get_data_parallel_rank
    assert Merak.MerakTrainer is merak_b200.MerakTrainer
    # a single-source path is the module itself, also below a package and by prefix translation
    import Merak.core.printer.timer as alias_timer
    import merak_b200.printer.timer as real_timer
    assert alias_timer is real_timer and real_timer.__name__ == "merak_b200.printer.timer"
    assert sys.modules["Merak.core.printer"] is sys.modules["merak_b200.printer"]
    from Merak.merak_args.args import MerakArguments
    assert MerakArguments is merak_b200.MerakArguments
    from Merak.core.mpu.layers import ColumnParallelLinear
    from merak_b200.parallel.layers import ColumnParallelLinear as real_col
    assert ColumnParallelLinear is real_col
    # attribute access from the top without an explicit sub-import
    assert Merak.core.mpu is mpu and Merak.utils.datasets.DynamicGenDataset is not None


def test_unknown_reference_path_is_a_missing_module():
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("Merak.core.does_not_exist")
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("Merak.core.printer.nothing")
    with pytest.raises(ImportError):
        exec("from Merak.core.mpu import no_such_name")


def test_reference_style_script_runs(tmp_path):
    """A script with the reference examples' import block and call sequence
    (examples/models/gpt2/run_gpt.py:24-75 of the reference) trains through the alias package."""
    import os
    import subprocess
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "run.py"
    script.write_text(textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        import Merak
        from Merak import MerakArguments, MerakTrainer, print_rank_0, init_empty_weights
        from Merak.utils.datasets import DynamicGenDataset
        from Merak.core import mpu
        from transformers import GPT2Config, GPT2LMHeadModel

        Merak.init(1, 1, 1, backend="gloo")
        args = MerakArguments(output_dir=%r, per_device_train_batch_size=2, gradient_accumulation_steps=2, max_steps=2,
                              logging_steps=1, no_cuda=True, report_to="none")
        config = GPT2Config(n_layer=2, n_embd=64, n_head=4, n_positions=64, vocab_size=512, resid_pdrop=0.0,
                            embd_pdrop=0.0, attn_pdrop=0.0)
        with init_empty_weights():
            probe = GPT2LMHeadModel(config)
        assert probe.transformer.wte.weight.is_meta          # the large tables and matrices hold no memory
        model = GPT2LMHeadModel(config)
        dataset = DynamicGenDataset(config, mode="text_only", dataset_size=32, seq_length=32)
        trainer = MerakTrainer(model=model, args=args, train_dataset=dataset)
        trainer.train()
        print_rank_0("dp rank %%d done" %% mpu.get_data_parallel_rank())
    """ % (root, str(tmp_path))))
    env = dict(os.environ, MERAK_QUIET="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29000 + (os.getpid() + 31) % 1000),
               RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-3000:]
    assert "steps: 2 loss:" in out and "dp rank 0 done" in out


def test_reference_style_trainer_subclass(tmp_path):
    """A trainer subclass with the reference's hook signatures (examples/bert_pretraining/run_bert.py:90-145 of
    the reference: ``create_dataloader(self)`` that sets ``self.train_dataloader``, ``create_optimizer(self,
    opt_model)`` that groups ``opt_model.named_parameters()``, ``create_lr_scheduler``, ``get_loss_fn``) trains."""
    import os
    import subprocess
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "run.py"
    script.write_text(textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        import torch
        import Merak
        from Merak import MerakArguments, MerakTrainer
        from Merak.core import mpu
        from Merak.utils import WorkerInitObj
        from Merak.utils.datasets import DynamicGenDataset
        from transformers import BertConfig, BertForMaskedLM

        Merak.init(1, 1, 1, backend="gloo")
        args = MerakArguments(output_dir=%r, per_device_train_batch_size=2, gradient_accumulation_steps=2, max_steps=3,
                              logging_steps=1, no_cuda=True, report_to="none", learning_rate=1e-3)
        config = BertConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, intermediate_size=128,
                            max_position_embeddings=64, vocab_size=512, return_dict=False,
                            hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
        model = BertForMaskedLM(config)
        calls = []

        class BertTrainer(MerakTrainer):
            def create_dataloader(self):
                sampler = torch.utils.data.RandomSampler(self.train_dataset)
                worker_init = WorkerInitObj(self.args.seed + mpu.get_data_parallel_rank())
                self.train_dataloader = torch.utils.data.DataLoader(
                    self.train_dataset, sampler=sampler, batch_size=self.args.per_device_train_batch_size,
                    num_workers=0, worker_init_fn=worker_init)
                calls.append("dataloader")

            def get_loss_fn(self):
                criterion = torch.nn.CrossEntropyLoss(ignore_index=-100)
                def loss_fn(outputs, labels):
                    logits = outputs[0] if isinstance(outputs, (tuple, list)) else outputs
                    return criterion(logits.view(-1, logits.size(-1)).float(), labels.view(-1))
                return loss_fn

            def create_optimizer(self, opt_model):
                named = list(opt_model.named_parameters())
                assert named and len({id(p) for _, p in named}) == len(named)
                no_decay = ["bias", "LayerNorm"]
                groups = [{"params": [p for n, p in named if not any(nd in n for nd in no_decay)], "weight_decay": 0.01},
                          {"params": [p for n, p in named if any(nd in n for nd in no_decay)], "weight_decay": 0.0}]
                assert groups[0]["params"] and groups[1]["params"]
                calls.append("optimizer")
                return torch.optim.AdamW(groups, lr=self.args.learning_rate)

            def create_lr_scheduler(self, optimizer):
                calls.append("scheduler")
                return torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: 1.0)

        dataset = DynamicGenDataset(config, mode="text_only", dataset_size=32, seq_length=32)
        trainer = BertTrainer(model=model, args=args, train_dataset=dataset)
        trainer.train()
        assert calls == ["dataloader", "optimizer", "scheduler"], calls
        assert isinstance(trainer.engine.optimizer, torch.optim.AdamW)
        print("hooks ok")
    """ % (root, str(tmp_path))))
    env = dict(os.environ, MERAK_QUIET="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29000 + (os.getpid() + 47) % 1000),
               RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-3000:]
    assert "steps: 3 loss:" in out and "hooks ok" in out
