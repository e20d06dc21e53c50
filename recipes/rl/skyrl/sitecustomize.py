"""Start-up hook: registers the recipe environments in every interpreter that has this directory on ``PYTHONPATH``.

Python imports a module named ``sitecustomize`` at start-up when one is on the path.  SkyRL scores rollouts in worker
processes that are started fresh (``multiprocessing`` spawn, Ray tasks); they do not inherit the driver's registered
environments, so ``skyrl_gym.make("bird_sql_arctic")`` there would fail with an unknown id.  Putting
``recipes/rl/skyrl`` on ``PYTHONPATH`` (the launchers under this directory do) makes every such process register
the environments before it does anything else.  Without ``skyrl_gym`` the hook does nothing; a failure here never
stops the interpreter.  Counterpart of recipes/rl/skyrl/*/sitecustomize.py in the reference.
"""
try:
    from recipes.rl.skyrl.envs import register_envs
    register_envs()
except Exception:           # not importable from this interpreter's path: leave start-up alone
    pass
