"""Classification and regression metrics on a toy prediction. Reference: examples/metrics_example.cpp."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tnn_b200.nn import metrics as M  # noqa: E402

torch.manual_seed(0)
labels = torch.randint(0, 5, (64,))
logits = torch.randn(64, 5) + 2.0 * torch.nn.functional.one_hot(labels, 5)
print("accuracy       ", round(M.accuracy(logits, labels), 4))
print("top-2 accuracy ", round(M.top_k_accuracy(logits, labels, 2), 4))
print("macro precision", round(float(M.precision(logits, labels, 5)), 4))
print("macro recall   ", round(float(M.recall(logits, labels, 5)), 4))
print("macro F1       ", round(float(M.f1_score(logits, labels, 5)), 4))
print("per-class F1   ", [round(float(v), 3) for v in M.f1_score(logits, labels, 5, macro=False)])
ce = float(torch.nn.functional.cross_entropy(logits, labels))
print("perplexity     ", round(M.perplexity(ce), 4))
y, t = torch.randn(100), torch.randn(100)
print("MAE / MSE / RMSE", round(M.mae(y, t), 4), round(M.mse(y, t), 4), round(M.rmse(y, t), 4))
