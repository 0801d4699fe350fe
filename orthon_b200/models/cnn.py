"""Small CNN for 3x32x32 images: conv3x3 3->32 s1 p1, conv3x3 32->64 s2 p1, conv3x3 64->128 s2
p1 (ReLU after each), spatial mean, Linear 128->10.
(reference project: examples/cifar10_cnn.py:18-90)"""
from .. import nn


class SmallCNN(nn.Module):
    def __init__(self, num_classes=10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 32, 3, stride=1, padding=1)
        self.conv2 = nn.Conv2d(32, 64, 3, stride=2, padding=1)
        self.conv3 = nn.Conv2d(64, 128, 3, stride=2, padding=1)
        self.head = nn.Linear(128, num_classes)

    def forward(self, x):
        h = self.conv1(x).relu()
        h = self.conv2(h).relu()
        h = self.conv3(h).relu()
        h = h.mean(3).mean(2)  # spatial mean -> [N, 128]
        return self.head(h)
