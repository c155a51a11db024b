"""poot_b200: a Blackwell-native LLM inference engine.

Layers (bottom up): ``tensor`` / ``target`` (dtypes, device description) -> ``quant`` / ``load`` / ``weights`` (storage
formats, checkpoints, roles) -> ``ir`` / ``oracle`` / ``plan`` (primitive graph, CPU reference evaluation, planner) ->
``models`` (family tracers and registry) -> ``ops`` / ``runtime`` / ``parallel`` (kernel bindings, device engine,
tensor / expert parallel communication) -> ``driver`` / ``llm`` / ``cli`` / ``serve`` (serving driver, public facade,
command line, HTTP server) with ``text`` (tokenizers, templates, guided decoding) and ``profile`` beside them.

``from poot_b200 import LLM, SamplingParams`` is the call a user makes; everything heavier is imported on demand so
that the CPU-only parts (graph, oracle, planner, loaders, server logic) work without a GPU.
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM
        return LLM
    if name == "SamplingParams":
        from .driver.sampler import SamplingParams
        return SamplingParams
    raise AttributeError(name)
