"""A parallel decoder block: ONE norm feeds the mixer and the feed-forward, and x <- x + (mixer(h) + ff(h)).  The block returns
the two sublayer outputs; the worker folds their sum into the fp32 residual together with the NEXT block's norm (one kernel)."""
from swiftllm_b200.worker.layers.feed_forward import build_feed_forward
from swiftllm_b200.model_config import LatentAttentionSpec, WindowAttentionSpec
from swiftllm_b200.worker.layers.latent_attention import LatentAttentionMixer
from swiftllm_b200.worker.layers.window_attention import WindowAttentionMixer

_MIXERS = {LatentAttentionSpec: LatentAttentionMixer, WindowAttentionSpec: WindowAttentionMixer}


class ParallelBlockLayer:
    def __init__(self, model_config, weight, layer_id: int):
        self.layer_id, self.weight = layer_id, weight
        spec = model_config.mixers[layer_id]
        self.mixer = _MIXERS[type(spec)](spec, weight, model_config.rms_norm_eps, model_config.cache_slot[layer_id])
        self.ff = build_feed_forward(model_config.ffs[layer_id], weight)

    def forward(self, h, caches, block_table, infer_state):
        y_mix = self.mixer.forward(h, caches, block_table, infer_state)
        y_ff = self.ff.forward(h) if self.ff is not None else None
        return y_mix, y_ff
