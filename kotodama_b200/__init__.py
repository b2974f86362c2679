"""kotodama-b200: a Blackwell-native pretraining and serving framework for the Kotodama
model family (Llama decoder + Block Attention Residuals, Muon + AdamW)."""
from .config import MODEL_PRESETS, ModelConfig

__version__ = "0.1.0"
__all__ = ["ModelConfig", "MODEL_PRESETS", "__version__"]
