from .instinct import Instinct, SurpriseAdamW   # noqa: F401
from .muon import MuonAdamW   # noqa: F401
from .experience import ExperienceOpt   # noqa: F401
