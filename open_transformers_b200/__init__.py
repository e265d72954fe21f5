"""B200-native bitwise-reproducible pretraining and audit-replay framework."""
__version__ = "0.1.0"
