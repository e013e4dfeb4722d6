"""Audio frontends: mel filterbank, log-mel from raw audio, SpecAugment."""

from .mel import *
from .specaugment import *
