// Shim: the host/device inline marker used by the pinned headers.
#pragma once
#ifndef HDI
#define HDI inline
#endif
