"""inferflux_b200: a single-GPU inference engine for the Qwen2.5 dense decoder,
written for B200 (sm_100a)."""
__version__ = "0.1.0"
