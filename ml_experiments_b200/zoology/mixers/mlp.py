"""State mixers: ``MLP`` and the gated ``GLU`` (zoology/mixers/mlp.py:5-50)."""
import torch.nn.functional as F
from torch import nn


class MLP(nn.Module):
    def __init__(self, d_model: int, hidden_mult: int = 1, activation=F.gelu, return_residual: bool = False, **kwargs):
        super().__init__()
        self.return_residual, self.activation = return_residual, activation
        self.fc1 = nn.Linear(d_model, d_model * hidden_mult)
        self.fc2 = nn.Linear(d_model * hidden_mult, d_model)

    def forward(self, x):
        y = self.fc2(self.activation(self.fc1(x)))
        return (y, x) if self.return_residual else y


class GLU(nn.Module):
    def __init__(self, d_model: int, hidden_mult: int = 1, activation=F.gelu, return_residual: bool = False, **kwargs):
        super().__init__()
        self.return_residual, self.activation = return_residual, activation
        self.fc1 = nn.Linear(d_model, d_model * hidden_mult)
        self.fc2 = nn.Linear(d_model, d_model * hidden_mult)
        self.fc3 = nn.Linear(d_model * hidden_mult, d_model)

    def forward(self, x):
        y = self.fc3(self.fc1(x) * self.activation(self.fc2(x)))
        return (y, x) if self.return_residual else y
