"""tinyinfer_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200."""
__version__ = "0.1.0"
