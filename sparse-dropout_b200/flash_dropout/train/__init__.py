"""Consumers of the SparseDrop layers (the reference's MLP and char-level GPT, eval/mlp/model.py and
eval/llm/model.py) and the data-parallel training step that runs them on 1..8 GPUs."""
from .dp import FlatGradDataParallel, GraphedTrainStep, train_step
from .models import GPT, BasicNet
