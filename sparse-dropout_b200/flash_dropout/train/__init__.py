"""Consumers of the SparseDrop layers that BASELINE's training-step workloads name (an MLP and a
char-level GPT) and the data-parallel step that runs them on 1..8 GPUs."""
from .dp import FlatGradDataParallel, GraphedTrainStep, train_step
from .models import GPT, BasicNet
