from rl_b200.evals.eval import eval_cons_k, eval_pass_k, run_env_eval  # noqa: F401
