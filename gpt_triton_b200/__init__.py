"""B200-native GPT-2 forward engine: hand-written sm_100a kernels behind the operator and
module surface of thevasudevgupta/gpt-triton.

Importing ``gpt_triton_b200.kernels`` / ``gpt_triton_b200.gpt`` loads ``libb200gpt.so`` and fails
loudly when it has not been built (``python -m gpt_triton_b200.build``); there is no fallback path.
"""

__all__ = ["kernels", "gpt", "build", "sharding"]
