from .instinct import Instinct, SurpriseAdamW   # noqa: F401
