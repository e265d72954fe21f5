"""`hydra.core.global_hydra.GlobalHydra`: the process-wide composition state (config/load.py:62-63)."""


class GlobalHydra:
    _instance = None

    def __init__(self) -> None:
        self.config_dir = None

    @classmethod
    def instance(cls) -> "GlobalHydra":
        if cls._instance is None:
            cls._instance = GlobalHydra()
        return cls._instance

    def is_initialized(self) -> bool:
        return self.config_dir is not None

    def clear(self) -> None:
        self.config_dir = None
