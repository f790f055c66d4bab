"""Consumers of the SparseDrop layers (the reference's MLP, char-level GPT and ViT, eval/mlp/model.py,
eval/llm/model.py and eval/vit/model.py) and the data-parallel training step that runs them on 1..8 GPUs."""
from .dp import FlatGradDataParallel, GraphedTrainStep, train_step
from .models import GPT, BasicNet, ViT
