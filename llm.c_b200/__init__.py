"""llm.c_b200: a Blackwell (sm_100a) native GPT-2 / GPT-3 pretraining framework.

PyTorch is the framework layer (tensors, streams, process groups, orchestration); every hot
operator is a hand-written CUDA kernel reached through ctypes (``ops``), the host runtime
(data loading, RNG, tokenizer, schedules, checkpoint IO) is a C++ library (``utils``), and the
ZeRO-1 communication path runs inside kernels over NVLink peer memory (``parallel``).
"""
__version__ = "0.1.0"
