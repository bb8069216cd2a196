from .engine import EngineArgs
from .model import InitArgs, InternalModelConfig, PeftArgs, TrainerArgs, get_model_config
from .openai_server import OpenAIServerConfig, ServerArgs, get_openai_server_config
from .train import TrainConfig

__all__ = [
    "EngineArgs", "get_model_config", "InternalModelConfig", "InitArgs", "PeftArgs", "TrainerArgs",
    "get_openai_server_config", "OpenAIServerConfig", "ServerArgs", "TrainConfig",
]
