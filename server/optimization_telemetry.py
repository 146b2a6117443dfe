from inferencehackathon_b200.serve.optimization_telemetry import *  # noqa: F401,F403
