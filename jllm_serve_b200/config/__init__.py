"""Typed configuration and the architecture registry."""
from .specs import (AttentionNames, ConfigError, Core, Decoder, DenseGluSpec, DenseMlpSpec, FeedForwardSpec, MatrixMemorySpec,
                    SelectiveStateSpaceSpec, FixedDecayLinearAttentionSpec,
                    GatedLinearAttentionSpec, GqaAttentionSpec, LatentAttentionSpec, LayerNames, LayerRun, LayerSpec, ModelNames,
                    MixerSpec, NormSpec, ParallelMixersSpec, RopeScaling, RopeTableSpec, RoutedExpertsSpec)
from .reader import ConfigReader
from .registry import (architecture_entry, load_config, model_type_of, parse_config, register_architecture, supported_architectures,
                       unregister_architecture)
from .families import DecoderDraft, parse_qwen3, parse_rope_scaling
from .madevik import parse_madevik
from .movivik import parse_movivik
from .bozevik import parse_bozevik
from .guvolix import parse_guvolix

register_architecture("qwen3", parse_qwen3, replace=True)
register_architecture("Madevik", parse_madevik, replace=True)
register_architecture("Movivik", parse_movivik, replace=True)
register_architecture("Bozevik", parse_bozevik, replace=True)
register_architecture("Guvolix", parse_guvolix, replace=True)
