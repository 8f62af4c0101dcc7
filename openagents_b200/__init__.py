"""openagents_b200: a Blackwell-native LLM serving and training framework.

Layers, top to bottom: ``gateway`` (provider seam, router, telemetry), ``serve`` (OpenAI-compatible
server, sessions, scheduler), ``train`` (data-parallel trainer, checkpoints, run/window state
machine), ``control`` (training control-plane predicates), ``models`` (llama, gpt2, gpt-oss),
``parallel`` (symmetric heap, tensor/expert/data parallel plans), ``ops`` (Python faces of the
sm_100a kernels), ``gguf`` (container and block formats) and ``oracle`` (CPU reference math).
"""
__version__ = "0.1.0"

ENGINE_NAME = "b200"
