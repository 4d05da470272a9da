"""A plain ``torch.nn`` image classifier (no framework layers, no Hugging Face config) through the
generic ``torch.fx`` tracing path and pipeline parallelism (the reference's examples/torch-models/
run_torchvision.py:40-66 with a torchvision ResNet; the network here is defined in this file so the
example has no extra dependency)."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from _common import degrees, parse

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import Dataset

import merak_b200 as Merak


class Block(nn.Module):
    def __init__(self, c_in, c_out, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(c_in, c_out, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(c_out)
        self.conv2 = nn.Conv2d(c_out, c_out, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(c_out)
        self.down = None if (stride == 1 and c_in == c_out) else nn.Sequential(
            nn.Conv2d(c_in, c_out, 1, stride, bias=False), nn.BatchNorm2d(c_out))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + (x if self.down is None else self.down(x)))


class ResNet(nn.Module):
    def __init__(self, widths=(64, 128, 256, 512), depth=2, num_classes=1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, widths[0], 7, 2, 3, bias=False), nn.BatchNorm2d(widths[0]), nn.ReLU(),
                                  nn.MaxPool2d(3, 2, 1))
        blocks, c = [], widths[0]
        for i, w in enumerate(widths):
            for j in range(depth):
                blocks.append(Block(c, w, 2 if (j == 0 and i > 0) else 1))
                c = w
        self.blocks = nn.Sequential(*blocks)
        self.fc = nn.Linear(c, num_classes)

    def forward(self, pixel_values):
        x = self.blocks(self.stem(pixel_values))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


class RandomImages(Dataset):
    def __init__(self, n, size, classes):
        self.n, self.size, self.classes = n, size, classes

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(i)
        return {"pixel_values": torch.randn(3, self.size, self.size, generator=g),
                "labels": torch.randint(0, self.classes, (), generator=g)}


def main():
    args, own = parse({"image_size": 224, "dataset_size": 1024, "width": 64, "num_classes": 1000})
    Merak.init(**degrees())
    w = own.width
    model = ResNet((w, 2 * w, 4 * w, 8 * w), num_classes=own.num_classes)
    args.input_names = ["pixel_values"]
    trainer = Merak.MerakTrainer(model, args, train_dataset=RandomImages(own.dataset_size, own.image_size, own.num_classes),
                                 loss_fn=lambda out, labels: F.cross_entropy(out.float(), labels))
    trainer.train()


if __name__ == "__main__":
    main()
