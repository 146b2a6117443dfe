"""Import-path shim: the reference is started with ``uvicorn server.main:app``; the implementation lives in
``inferencehackathon_b200.serve``."""
