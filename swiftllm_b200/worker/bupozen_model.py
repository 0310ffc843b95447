"""BupozenModel - worker of the Bupozen design: parallel blocks of latent attention + dense / mixture-of-experts squared-ReLU
feed-forwards on an fp32 residual stream.  Everything but the configuration, the weights and the kernel sources is the shared
parallel-block worker (worker/parallel_block_model.py)."""
from swiftllm_b200.model_config import BupozenModelConfig
from swiftllm_b200.worker.parallel_block_model import ParallelBlockModel
from swiftllm_b200.worker.weight import load_bupozen_weights


class BupozenModel(ParallelBlockModel):
    NATIVE_SOURCES = ParallelBlockModel.NATIVE_SOURCES + ("latent_attn.cu",)
    CONFIG_CLASS = BupozenModelConfig

    @staticmethod
    def _load_weights(model_config, dtype, model_path, use_dummy, getter, device):
        return load_bupozen_weights(model_config, dtype, model_path, use_dummy, getter=getter, device=device)
