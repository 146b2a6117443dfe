from inferencehackathon_b200.serve.app import create_app

app = create_app()
