"""Model families (GPT-2, Llama, Mistral, Gemma-2, Kepovik, Repudra, Lonulix, Fisopel): configs, weights, torch oracle, native pieces."""
from .config import PRESETS, ModelConfig, resolve_config, split_layers  # noqa: F401


def piece_class(cfg: ModelConfig):
    """The GPU piece implementation that serves ``cfg``: uniform softmax-attention decoders run on ``NativePiece``,
    configs with per-layer mixer specs (sigmoid attention / delta rule with residual streams; parallel blocks; post-norm
    layers with latent attention, HGRN2 and routed experts; looped parallel blocks with a norm per sublayer) on ``HybridPiece``."""
    if cfg.hybrid:
        from .hybrid import HybridPiece
        return HybridPiece
    from .native import NativePiece
    return NativePiece
