"""Speech2Text speech translation (examples/models/speech2text): the Hugging Face ``Speech2TextForConditionalGeneration`` with random weights on generated data.

    torchrun --nproc_per_node=4 --master-addr 127.0.0.1 examples/models/speech2text/run_speech2text.py \\
        --output_dir ./out --per_device_train_batch_size 4 --gradient_accumulation_steps 4 --max_steps 50
    PP=2 TP=2 ...   (degrees come from the environment; ``--tiny 1`` shrinks the model for a CPU run)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import transformers as T  # noqa: E402
from _hf import run  # noqa: E402

TINY_S2T = dict(max_source_positions=64, max_target_positions=64, num_conv_layers=2, conv_kernel_sizes=(5, 5),
                conv_channels=32, input_feat_per_channel=80, pad_token_id=0, decoder_start_token_id=0, eos_token_id=1)


if __name__ == "__main__":
    run(T.Speech2TextConfig, T.Speech2TextForConditionalGeneration, mode="speech2text", tiny_overrides=TINY_S2T)   # features arrive as [frames, filter banks]
