"""fllm_b200: a Blackwell-native (B200, sm_100a) LLM inference engine.

Layers, bottom to top: ``formats`` (GGUF / safetensors, packed weights stay packed),
``ops`` (hand-written CUDA kernels behind ``torch.ops.fllm_b200``), ``comm``
(peer-memory collectives), ``parallel`` (TP x PP x EP layout and sharding),
``models`` (decoder runners), ``runtime`` (paged KV, scheduler, engine),
``server`` (OpenAI / Anthropic / Ollama dialects) and ``cli``.
"""
__version__ = "0.1.0"
