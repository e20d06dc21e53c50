"""Single-turn text environments for the SkyRL recipes: one model response in, one reward out, episode done.

``extras`` is the dataset row as SkyRL's prompt dataset forwards it; both verl-format (``reward_model.ground_truth``)
and SkyRL-format (``reward_spec.ground_truth``) rows work.  With ``skyrl_gym`` installed the classes derive from its
``BaseTextEnv`` and :func:`register_envs` adds them to its registry (ids ``gsm8k_arctic``, ``bird_sql_arctic``,
``long_context_qa``); without it they are plain classes with the same ``step`` contract, which is what the offline
loop in ``run_loop.py`` and the tests use.  Counterpart of recipes/rl/skyrl/long_context_qa/arctic_rl/envs/ in the
reference."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

from ..rewards.bird_reward import bird_reward
from ..rewards.gsm8k_reward import gsm8k_reward
from ..rewards.long_context_qa_reward import long_context_qa_reward

try:                                            # pragma: no cover - depends on the SkyRL checkout
    from skyrl_gym.envs.base_text_env import BaseTextEnv, BaseTextEnvStepOutput
    HAVE_SKYRL_GYM = True
except ImportError:
    HAVE_SKYRL_GYM = False

    class BaseTextEnv:                          # the two members the environments rely on
        def __init__(self) -> None:
            self.turns = 0

    @dataclass
    class BaseTextEnvStepOutput:
        observations: List[Any] = field(default_factory=list)
        reward: float = 0.0
        done: bool = True
        metadata: Dict[str, Any] = field(default_factory=dict)


def _ground_truth(extras: Dict[str, Any], env: str):
    block = extras.get("reward_model") or extras.get("reward_spec") or {}
    gt = block.get("ground_truth")
    if gt is None:
        raise ValueError(f"{env} needs reward_model.ground_truth (or reward_spec.ground_truth) in the dataset row")
    return gt


class _SingleTurnEnv(BaseTextEnv):
    name = "single_turn"

    def __init__(self, env_config: Any = None, extras: Dict[str, Any] = None):
        super().__init__()
        extras = dict(extras or {})
        self.ground_truth = _ground_truth(extras, type(self).__name__)
        self.extra_info: Dict[str, Any] = dict(extras.get("extra_info") or {})
        self.data_source: str = extras.get("data_source", self.name)
        self.env_config = env_config

    def reward(self, response: str) -> float:
        raise NotImplementedError

    def step(self, action: str) -> BaseTextEnvStepOutput:
        return BaseTextEnvStepOutput(observations=[], reward=float(self.reward(action)), done=True, metadata={})


class GSM8KEnv(_SingleTurnEnv):
    name = "gsm8k"

    def reward(self, response: str) -> float:
        return gsm8k_reward(response, str(self.ground_truth), method="flexible", format_score=0.0)


class BirdSQLEnv(_SingleTurnEnv):
    """Executes the model's SQL and the gold SQL against ``extra_info.db_path`` and compares the result sets."""
    name = "bird"

    def reward(self, response: str) -> float:
        db_path = self.extra_info.get("db_path")
        if not db_path:
            raise ValueError("BirdSQLEnv needs extra_info.db_path (written by preprocess_bird.py)")
        return bird_reward(response, str(self.ground_truth), db_path)


class LongContextQAEnv(_SingleTurnEnv):
    name = "long_context_qa"

    def reward(self, response: str) -> float:
        gold = self.ground_truth if isinstance(self.ground_truth, (list, tuple)) else [self.ground_truth]
        return long_context_qa_reward(response, [str(g) for g in gold])


ENVS = {"gsm8k_arctic": GSM8KEnv, "bird_sql_arctic": BirdSQLEnv, "long_context_qa": LongContextQAEnv}


def make(env_id: str, extras: Dict[str, Any], env_config: Any = None) -> _SingleTurnEnv:
    if env_id not in ENVS:
        raise KeyError(f"unknown environment {env_id!r} (known: {sorted(ENVS)})")
    return ENVS[env_id](env_config, extras)


def register_envs() -> List[str]:
    """Adds the environments to ``skyrl_gym``'s registry (ids already present are left alone).  Returns the ids
    registered by this call; an empty list without ``skyrl_gym``."""
    if not HAVE_SKYRL_GYM:
        return []
    from skyrl_gym.envs.registration import register          # pragma: no cover
    done = []                                                  # pragma: no cover
    for env_id, cls in ENVS.items():                           # pragma: no cover
        try:
            register(id=env_id, entry_point=f"{__name__}:{cls.__name__}")
            done.append(env_id)
        except Exception:                                      # already registered by another import of this module
            pass
    return done                                                # pragma: no cover
