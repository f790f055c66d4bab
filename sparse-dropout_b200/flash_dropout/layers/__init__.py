from .dropout_conv import DropoutConv2d
from .dropout_mm import DropoutMM
