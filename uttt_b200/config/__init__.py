from .lm_config import (CONFIG_REGISTRY, LMConfig, UTTTMoEConfig, UTTTDenseConfig, TTTMoEConfig,
                        TTTMoENoLBConfig, TTTDenseConfig, LaCTConfig, TransformerConfig, SWAMixerConfig,
                        config_from_dict, load_config, named_config)
