"""The Python entry point: ``LLM(model_dir, ...).generate(prompts, sampling_params)``.

The reference exposes ``LLMEngine(ModelRunner(model, ecfg)).add_request(...)`` and
``run_until_complete()`` (src/qwen25vl_lite/engine.py:507,878; tests/test_engine.py:50-51);
``LLM`` wraps the same three calls and keeps the engine's option names
(``num_blocks``, ``block_size``, ``max_num_seqs``, ``max_num_batched_tokens``,
``max_model_len``, ``enable_chunked_prefill``, ``dtype``).
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model
from ..weights.random_init import load_random_model
from .runner import ModelRunner
from .scheduler import LLMEngine, RequestOutput


class LLM:
    def __init__(self, model: Optional[str] = None, *, dtype: str = "bfloat16", device: str = "cuda:0",
                 engine_config: Optional[EngineConfig] = None, random_config: Optional[dict] = None,
                 weights_seed: int = 0, **engine_options):
        """``model``: a folder with config.json and safetensors.  ``random_config`` (a
        config.json as a dict) with ``weights_seed`` instead builds the model with random
        weights drawn on the device.  Other keyword options are ``EngineConfig`` fields."""
        self.ecfg = engine_config or EngineConfig(dtype=dtype, device=device, **engine_options)
        if model is not None:
            self.config, self.model = load_model(model, self.ecfg.dtype, self.ecfg.device)
        elif random_config is not None:
            self.config, self.model = load_random_model(random_config, weights_seed, self.ecfg.dtype, self.ecfg.device)
        else:
            raise ValueError("LLM needs a model folder or a random_config")
        self.runner = ModelRunner(self.model, self.ecfg.num_blocks, self.ecfg.block_size, self.ecfg.max_num_seqs,
                                  max_step_tokens=self.ecfg.max_num_batched_tokens, cuda_graphs=self.ecfg.cuda_graph)
        self.sampler = Sampler(self.ecfg.device)
        self.engine = LLMEngine(self.runner, self.sampler, self.ecfg, getattr(self.config, "eos_token_id", None))

    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 positions: Optional[Sequence] = None) -> List[RequestOutput]:
        """Generates for every prompt (lists of token ids) and returns the outputs in the
        order of the prompts.  ``positions[i]`` may give prompt i explicit position ids."""
        if prompt_token_ids and isinstance(prompt_token_ids[0], int):
            prompt_token_ids = [prompt_token_ids]
        n = len(prompt_token_ids)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * n
        if len(sampling_params) != n:
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.engine.add_request(p, sp, positions=None if positions is None else positions[i])
               for i, (p, sp) in enumerate(zip(prompt_token_ids, sampling_params))]
        before = len(self.engine.finished)
        self.engine.run_until_complete()
        by_id = {o.seq_id: o for o in self.engine.finished[before:]}
        return [by_id[i] for i in ids]
