"""hibana_b200: a Blackwell-datacenter (B200, sm_100a) native LLM inference engine.

Package map: ``config`` / ``target`` (settings and model presets), ``ops`` (hand-written sm_100a kernels behind
plain-PyTorch references), ``models`` (layer library and model families), ``cache`` (paged KV + recurrent
state pools, radix prefix cache, SSD tier), ``engine`` (scheduler, executor, speculation, CUDA graphs),
``parallel`` (NVLink peer-memory communicator, TP / EP / DP), ``weights`` (NVFP4 / FP8 / w3 checkpoints),
``api`` and ``cli`` (OpenAI / Anthropic HTTP surface and the ``hibana`` command).
"""
__version__ = "0.1.0"
