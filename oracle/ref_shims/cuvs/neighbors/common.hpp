// Shim: the pinned reference headers include this file but need nothing from it.
#pragma once
