"""VGG16 (configuration D, no batch norm) written out in torch.nn: the 32
trainable tensors / 138,357,544 parameters of the reference's vgg16 gradient
set (testdata/vgg16.txt there).  torchvision is not needed."""
import torch
from torch import nn


class VGG16(nn.Module):
    def __init__(self, num_classes=1000):
        super().__init__()
        layers, cin = [], 3
        for v in (64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M",
                  512, 512, 512, "M"):
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers += [nn.Conv2d(cin, v, 3, padding=1), nn.ReLU(inplace=True)]
                cin = v
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d(7)
        self.classifier = nn.Sequential(
            nn.Linear(512 * 7 * 7, 4096), nn.ReLU(inplace=True), nn.Dropout(),
            nn.Linear(4096, 4096), nn.ReLU(inplace=True), nn.Dropout(),
            nn.Linear(4096, num_classes))

    def forward(self, x):
        x = self.avgpool(self.features(x))
        return self.classifier(torch.flatten(x, 1))
