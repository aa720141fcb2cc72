from streamep_b200.utils.nvlink import check_nvlink_connections  # noqa: F401
