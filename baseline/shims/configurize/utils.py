from steptronoss_b200.config.mock_imports import get_object_from_file  # noqa: F401
