"""RSA helpers for secrets kept in job configs (``recis/common/crypto_utils.py``): PKCS#1 v1.5 encryption with base64-encoded
DER keys, base64 text in and out. Built on the ``cryptography`` package (the reference uses PyCryptodome)."""
from __future__ import annotations

import base64


def encode(data, public_key, binary_code="utf-8") -> str:
    """Encrypt ``data`` with a base64-encoded DER (SubjectPublicKeyInfo) public key; returns base64 text."""
    from cryptography.hazmat.primitives import serialization
    from cryptography.hazmat.primitives.asymmetric import padding
    key = serialization.load_der_public_key(base64.b64decode(str(public_key)))
    return base64.b64encode(key.encrypt(str(data).encode(binary_code), padding.PKCS1v15())).decode(binary_code)


def decode(data, private_key, binary_code="utf-8") -> str:
    """Decrypt base64 text produced by ``encode`` with a base64-encoded DER (PKCS#8) private key."""
    from cryptography.hazmat.primitives import serialization
    from cryptography.hazmat.primitives.asymmetric import padding
    key = serialization.load_der_private_key(base64.b64decode(str(private_key)), password=None)
    return key.decrypt(base64.b64decode(str(data)), padding.PKCS1v15()).decode(binary_code)
