from .moe_block import MoEBlock, MoEConfig, CONFIGS, smoke_step

__all__ = ["MoEBlock", "MoEConfig", "CONFIGS", "smoke_step"]
