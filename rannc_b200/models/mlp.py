"""Tutorial-sized multi-layer perceptrons."""
import torch
import torch.nn as nn


class TutorialMLP(nn.Module):
    """Linear 512 -> 1024, ReLU, Linear 1024 -> 1024, ReLU, Linear 1024 -> 10."""

    def __init__(self, d_in: int = 512, hidden: int = 1024, classes: int = 10):
        super().__init__()
        self.fc1 = nn.Linear(d_in, hidden)
        self.fc2 = nn.Linear(hidden, hidden)
        self.fc3 = nn.Linear(hidden, classes)

    def forward(self, x):
        return self.fc3(torch.relu(self.fc2(torch.relu(self.fc1(x)))))


class TutorialMLPWithLoss(nn.Module):
    def __init__(self, **kw):
        super().__init__()
        self.net = TutorialMLP(**kw)

    def forward(self, x, y):
        return nn.functional.cross_entropy(self.net(x), y)


class DeepMLP(nn.Module):
    """``layers`` x Linear(hidden, hidden), the model of the reference's tutorial script."""

    def __init__(self, hidden: int = 512, layers: int = 10):
        super().__init__()
        self.layers = nn.ModuleList([nn.Linear(hidden, hidden) for _ in range(layers)])

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x
