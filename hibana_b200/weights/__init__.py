"""Checkpoint formats: ModelOpt NVFP4 / FP8 safetensors (modelopt.py, checkpoint.py) and the 3-bit copies (w3.py)."""
