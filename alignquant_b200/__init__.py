"""B200-native (sm_100a) implementation of AlignQuant's mixed W4/W8-A8 linear path."""

__version__ = "0.1.0"
