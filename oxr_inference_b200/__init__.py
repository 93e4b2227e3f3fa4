"""B200-native single-GPU inference engine for the Qwen3 dense decoder.

Layers, bottom to top: ``config`` (typed config.json + architecture registry), ``weights`` (safetensors
by tensor name, random-weights mode), ``ops`` + ``csrc`` (hand-written sm_100a kernels), ``parts``
(norm, position encoding, mixer, feed-forward, block, decoder), ``cache`` (paged KV with block tables,
per-request state slots), ``engine`` (step function, scheduler, CUDA-graph decode, ``Engine.generate``),
``sampling``.
"""

__version__ = "0.1.0"

from oxr_inference_b200.config import EngineSettings, load_model_config  # noqa: F401


def __getattr__(name: str):
    # Engine pulls in torch and the CUDA extension; import it lazily so that config-only users stay light.
    if name in ("Engine", "Completion", "SamplingParams", "Busy"):
        from oxr_inference_b200.engine import api

        return getattr(api, name)
    raise AttributeError(name)
