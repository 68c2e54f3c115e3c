"""Weight refit: moving the trainer's current weights into the generation engine's layout."""
from rl_b200.refit.plan import CopyOp, RefitPlan, build_refit_plan, serving_param_layout  # noqa: F401
