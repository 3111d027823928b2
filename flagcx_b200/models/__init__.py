"""flagcx_b200.models"""
