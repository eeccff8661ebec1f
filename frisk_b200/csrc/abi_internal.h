// Shared between the translation units of libfrisk_b200.so; not part of the C ABI.
#pragma once

// Sets the text frisk_b200_last_error() returns on the calling thread.
__attribute__((visibility("hidden"))) void frisk_internal_set_error(const char* text);
