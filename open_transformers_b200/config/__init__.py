from .load import compose, default_configs_dir, load_config, parse_config_resolved, resolve_to_typed
from .schema import (DataConfig, DataSourceConfig, GlobalBatchTokens, GradNormLogConfig, InitConfig, LoggingConfig,
                     ModelConfig, ModuleSelection, OptimConfig, QATConfig, RootConfig, RunConfig, ScheduleConfig,
                     SpikeConfig, StateHashConfig, TrainConfig, ZLossConfig)

__all__ = [n for n in dir() if not n.startswith("_")]
