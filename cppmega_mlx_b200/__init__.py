"""B200-native (sm_100a) training and serving framework with the capabilities of cppmega_mlx."""
__version__ = "0.1.0"
