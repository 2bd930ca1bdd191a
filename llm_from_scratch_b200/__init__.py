"""B200-native kernels and host layer for the continuous-batching prefill/decode step."""
__version__ = "0.1.0"
