from .checkpoint import CheckpointLoader, CheckpointSaver, rotate_checkpoints
from .utils import (ShardedSafetensorLoader, check_state_dict, detect_checkpoint_format, get_checkpoint_name,
                    get_zero_checkpoint_name, read_metadata)
