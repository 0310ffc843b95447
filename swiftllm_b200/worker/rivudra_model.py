"""RivudraModel - worker of the Rivudra design: parallel blocks of gated sliding-window attention (grouped key/value heads,
partial interleaved rotary, a softmax sink) + group-routed mixtures of clamped gated-linear-unit experts with a shared expert,
on an fp32 residual stream with a scaled embedding and norm weights stored around zero.  Everything but the configuration, the
weights and the kernel sources is the shared parallel-block worker (worker/parallel_block_model.py)."""
from swiftllm_b200.model_config import RivudraModelConfig
from swiftllm_b200.worker.parallel_block_model import ParallelBlockModel
from swiftllm_b200.worker.weight import load_rivudra_weights


class RivudraModel(ParallelBlockModel):
    NATIVE_SOURCES = ParallelBlockModel.NATIVE_SOURCES + ("window_attn.cu",)
    CONFIG_CLASS = RivudraModelConfig

    @staticmethod
    def _load_weights(model_config, dtype, model_path, use_dummy, getter, device):
        return load_rivudra_weights(model_config, dtype, model_path, use_dummy, getter=getter, device=device)
