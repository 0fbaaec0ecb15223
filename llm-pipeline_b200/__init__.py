"""B200-native inference engine for the Qwen3 dense decoder of DavidAkinpelu/llm-pipeline.

Sub-packages: ``config`` (typed configurations, architecture registry), ``weights`` (safetensors
loading, random model folders), ``parts`` (norm, position encoding, mixer, feed-forward, block),
``models`` (architectures assembled from parts), ``cache`` (paged keys/values, state slots),
``engine`` (step function, scheduler, generation), ``sampling``, ``ops`` (bindings of the CUDA
library built from ``csrc``).
"""

__version__ = "0.1.0"
