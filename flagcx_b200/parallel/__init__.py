"""flagcx_b200.parallel"""
