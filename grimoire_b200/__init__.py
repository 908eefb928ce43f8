"""grimoire_b200: a Blackwell-native LLM inference engine with GRIMOIRE's capabilities.

PyTorch is the framework layer (tensors, streams, CUDA graphs, torch.distributed/NCCL plumbing);
the hot paths are hand-written sm_100a kernels in ``csrc/kernels`` and the host runtime pieces
(codecs, readers, tokenizer, scheduler core) are C++ in ``csrc/host``.
"""

__version__ = "0.1.0"
