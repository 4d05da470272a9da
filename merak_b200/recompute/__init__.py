from .checkpointing import (CheckpointFunction, PreCheckpointFunction, RNGManager, RNGStatesTracker, checkpoint,
                            get_rng_tracker, model_parallel_manual_seed, pre_checkpoint, pending_recomputes,
                            run_pending_recomputes)

# name used by the reference API
model_parallel_cuda_manual_seed = model_parallel_manual_seed
