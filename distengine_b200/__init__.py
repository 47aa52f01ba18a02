"""distengine_b200: a single-GPU inference engine for the Llama decoder on B200 (sm_100a)."""

__version__ = "0.1.0"
