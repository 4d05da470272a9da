"""UNet segmentation model captured with ``torch.export`` (``--trace_method dynamo``) instead of
``torch.fx`` symbolic tracing, then split over pipeline stages (the reference's examples/unet/
run_unet.py:36-121 with the pytorch_unet submodule; the small UNet here is defined in this file)."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import Dataset

import merak_b200 as Merak


def double_conv(c_in, c_out):
    return nn.Sequential(nn.Conv2d(c_in, c_out, 3, padding=1), nn.GroupNorm(4, c_out), nn.ReLU(),
                         nn.Conv2d(c_out, c_out, 3, padding=1), nn.GroupNorm(4, c_out), nn.ReLU())


class UNet(nn.Module):
    def __init__(self, channels=3, classes=2, width=32):
        super().__init__()
        w = width
        self.inc, self.d1, self.d2 = double_conv(channels, w), double_conv(w, 2 * w), double_conv(2 * w, 4 * w)
        self.u1, self.u2 = double_conv(4 * w + 2 * w, 2 * w), double_conv(2 * w + w, w)
        self.outc = nn.Conv2d(w, classes, 1)

    def forward(self, pixel_values):
        x1 = self.inc(pixel_values)
        x2 = self.d1(F.max_pool2d(x1, 2))
        x3 = self.d2(F.max_pool2d(x2, 2))
        y = self.u1(torch.cat([F.interpolate(x3, scale_factor=2.0, mode="nearest"), x2], dim=1))
        y = self.u2(torch.cat([F.interpolate(y, scale_factor=2.0, mode="nearest"), x1], dim=1))
        return self.outc(y)


class RandomMasks(Dataset):
    def __init__(self, n, size, classes):
        self.n, self.size, self.classes = n, size, classes

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(i)
        return {"pixel_values": torch.randn(3, self.size, self.size, generator=g),
                "labels": torch.randint(0, self.classes, (self.size, self.size), generator=g)}


def main():
    args, own = parse({"image_size": 128, "width": 32, "classes": 2, "dataset_size": 512, "trace_method": "dynamo"})
    Merak.init(**degrees())
    model = UNet(3, own.classes, own.width)
    args.input_names = ["pixel_values"]
    trainer = Merak.MerakTrainer(model, args, train_dataset=RandomMasks(own.dataset_size, own.image_size, own.classes),
                                 loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
    trainer.train()


if __name__ == "__main__":
    main()
