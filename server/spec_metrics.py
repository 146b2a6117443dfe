from inferencehackathon_b200.serve.spec_metrics import *  # noqa: F401,F403
