from .base import (BuildContext, StepBatch, build_part, part_class, register_part, registered_parts,
                   unregister_part)
from . import rotary, norm, linear, attention, feed_forward, block, delta, latent, hyper   # registers the built-in parts
from .attention import GQAttention
from .block import PreNormResidualBlock
from .delta import GatedDeltaMixer
from .feed_forward import GatedSiluFeedForward, SquaredReluFeedForward
from .hyper import HyperConnectionBlock
from .latent import LatentAttention
from .linear import DenseLinear
from .norm import RMSNorm
from .rotary import NoPosition, RotaryHalfSplit
from . import ssm, recurrent, window_attention, parallel, moe   # more built-in parts
from .block import SublayerOutputNormBlock
from .moe import RoutedExperts
from .norm import LayerNorm
from .parallel import ParallelMixers
from .recurrent import GatedRecurrentMixer
from .ssm import StateSpaceMixer
from .window_attention import WindowAttention
from . import sigmoid_attention   # one more built-in mixer
from .block import SandwichNormBlock
from .feed_forward import XieluFeedForward
from .sigmoid_attention import SigmoidAttention
