from steptronoss_b200.config.mock_imports import mock_imports  # noqa: F401
