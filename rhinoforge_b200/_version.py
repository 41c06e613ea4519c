"""Distribution version and API level (the API level follows the reference's 5.x surface)."""
API_VERSION = "5.0.0"
DISTRIBUTION_VERSION = "0.1.0"

__all__ = ["API_VERSION", "DISTRIBUTION_VERSION"]
