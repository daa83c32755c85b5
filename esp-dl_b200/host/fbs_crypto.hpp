// AES-128 (encryption direction, as CTR mode needs) and SHA-256 for the model loader: encrypted .espdl payloads
// (esp-dl/fbs_loader/src/fbs_loader.cpp:86-124: AES-128-CTR, counter block starting at bytes 10..1F, big-endian
// increment) and the integrity digest of PDL3 packages (fbs_loader.cpp:664-770).  Plain restatements of FIPS-197 and
// FIPS 180-4; the reference takes both from mbedtls.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace fbs {

/// plaintext[i] = ciphertext[i] XOR keystream[i] (the same call encrypts and decrypts).
void aes128_ctr(const uint8_t *in, uint8_t *out, size_t size, const uint8_t key[16], const uint8_t nonce[16]);

class Sha256 {
public:
    Sha256();
    void update(const uint8_t *data, size_t size);
    void finish(uint8_t out[32]);

private:
    void block(const uint8_t *p);
    uint32_t m_h[8];
    uint8_t m_buf[64];
    size_t m_fill = 0;
    uint64_t m_bits = 0;
};

} // namespace fbs
